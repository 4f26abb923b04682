// qmv_i8_inst_e.cu — instantiations of the integer tensor-core affine_qmv kernel for J = 21 groups per warp
// (rows of 10752 codes over 8 warps).
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_w<21>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

}  // namespace lthn
