// Instances of the tcgen05 matrix product for many tokens on pairs of blocks (cta_group::2: 256 tokens x 192 or 256 features).
#include "gemm_tcgen05.cuh"

namespace ptl {

int launch_pair_tiles(int bn, int epi, const CUtensorMap& mr, const CUtensorMap& mc, const CUtensorMap& mo, const GemmParams& p, dim3 grid,
                      cudaStream_t s) {
  switch (bn) {
    case 192: return launch_epi<192, true>(epi, mr, mc, mo, p, grid, s);
    case 256: return launch_epi<256, true>(epi, mr, mc, mo, p, grid, s);
  }
  return fail("gemm_tc: no paired instance for tiles of %d features", bn);
}

}  // namespace ptl
