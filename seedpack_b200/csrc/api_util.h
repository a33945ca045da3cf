// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>

#include "../../include/seedgrow.h"

namespace sg {

// records the error text for sg_last_cuda_error() and maps to a status code
int cuda_ok(cudaError_t e);
// cudaSetDevice with error mapping
int use_device(int device);
// address of the device's status word (a __device__ int of the library, one per device)
int* status_word(int device);
// IQ grids / maps / neighbour lists installed on this device?
bool tables_ready(int device);

}  // namespace sg
