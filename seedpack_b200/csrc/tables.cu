// IQ grid tables (placeholder).
#include "api_util.h"
namespace sg { bool tables_ready(int) { return false; } }
