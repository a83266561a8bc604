// Decode kernel instantiations for patches of up to 4x4 blocks of 32 and rank up to 64.
#include "bqq_decode_kernel.cuh"
namespace bqq {
BQQ_DECODE_VARIANT(3, 4, 4, 2)
}
