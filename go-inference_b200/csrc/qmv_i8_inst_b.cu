// qmv_i8_inst_b.cu — instantiations of the integer tensor-core affine_qmv kernel for J = 4, 6, 7 groups per warp.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_w<4>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<6>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<7>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

}  // namespace lthn
