// Decode kernel instantiations for patches of up to 1x1 blocks of 32 and rank up to 32.
#include "bqq_decode_kernel.cuh"
namespace bqq {
BQQ_DECODE_VARIANT(0, 1, 1, 1)
}
