// qmv_i8_inst_b8.cu — instantiations of the integer tensor-core affine_qmv kernel for 8-bit codes, J = 2, 3, 4.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_b8<2>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_b8<3>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_b8<4>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
}  // namespace lthn
