// Instances of the tcgen05 matrix product for few tokens (operands swapped: 16, 32 or 64 token columns).
#include "gemm_tcgen05.cuh"

namespace ptl {

int launch_few_tokens(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                      cudaStream_t s) {
  switch (bn) {
    case 16: return launch_epi<16>(epi, mr, mc, mo, p, grid, s);
    case 32: return launch_epi<32>(epi, mr, mc, mo, p, grid, s);
    case 64: return launch_epi<64>(epi, mr, mc, mo, p, grid, s);
  }
  return fail("gemm_tc: no instance for %d token columns", bn);
}

}  // namespace ptl
