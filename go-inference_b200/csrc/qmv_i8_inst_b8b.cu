// qmv_i8_inst_b8b.cu — instantiations of the integer tensor-core affine_qmv kernel for 8-bit codes, J = 6, 9, 12.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_b8<6>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_b8<9>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_b8<12>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
}  // namespace lthn
