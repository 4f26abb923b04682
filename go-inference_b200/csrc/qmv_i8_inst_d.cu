// qmv_i8_inst_d.cu — instantiations of the integer tensor-core affine_qmv kernel for J = 12, 16, 18 groups per warp.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_w<12>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<16>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<18>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

}  // namespace lthn
