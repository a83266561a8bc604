// Decode kernel instantiations for patches of up to 2x2 blocks of 32 and rank up to 64.
#include "bqq_decode_kernel.cuh"
namespace bqq {
BQQ_DECODE_VARIANT(2, 2, 2, 2)
}
