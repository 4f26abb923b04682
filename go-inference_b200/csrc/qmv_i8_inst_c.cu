// qmv_i8_inst_c.cu — instantiations of the integer tensor-core affine_qmv kernel for J = 8, 9 groups per warp.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_w<8>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<9>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

}  // namespace lthn
