// Decode kernel instantiations for a batch tile of 4 row(s) of X.
#include "bqq_decode_kernel.cuh"
namespace bqq {
template int decode_launch_mt<4>(const DecodeParams&, const DecodePlan&, int, int, cudaStream_t);
}
