// The error text of the 'core' library.
#include "common.cuh"

PH_DEFINE_LAST_ERROR(ph_core)
