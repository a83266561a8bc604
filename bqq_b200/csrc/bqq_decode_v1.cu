// Decode kernel instantiations for patches of up to 2x2 blocks of 32 and rank up to 32.
#include "bqq_decode_kernel.cuh"
namespace bqq {
BQQ_DECODE_VARIANT(1, 2, 2, 1)
}
