// IQ quantisers (placeholder until the grid kernels land).
#pragma once
#include "search.cuh"
namespace sg {
static int dispatch_iq(int, int, bool, const Job&, int, cudaStream_t) { return SG_ERR_TYPE; }
}
