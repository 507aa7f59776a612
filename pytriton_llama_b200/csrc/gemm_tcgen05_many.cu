// Instances of the tcgen05 matrix product for many tokens (tiles of 128 tokens x 128, 192 or 256 features).
#include "gemm_tcgen05.cuh"

namespace ptl {

int launch_many_tokens(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                       cudaStream_t s) {
  switch (bn) {
    case 128: return launch_epi<128>(epi, mr, mc, mo, p, grid, s);
    case 192: return launch_epi<192>(epi, mr, mc, mo, p, grid, s);
    case 256: return launch_epi<256>(epi, mr, mc, mo, p, grid, s);
  }
  return fail("gemm_tc: no instance for tiles of %d features", bn);
}

}  // namespace ptl
