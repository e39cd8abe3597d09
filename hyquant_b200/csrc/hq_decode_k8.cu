// The decode kernel's instantiations for a 8-bit K prefix (V in 8, 4 and 2 bits); see hq_decode_kernel.cuh.
#include "hq_decode_kernel.cuh"

namespace hq {
HQ_DECODE_DEFINE(8, 8)
HQ_DECODE_DEFINE(8, 4)
HQ_DECODE_DEFINE(8, 2)
}  // namespace hq
