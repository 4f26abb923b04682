// qmv_i8_inst_a.cu — instantiations of the integer tensor-core affine_qmv kernel for J = 1, 2, 3 groups per warp.
#include "qmv_i8_kernel.cuh"

namespace lthn {
template int32_t launch_i8_w<1>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<2>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
template int32_t launch_i8_w<3>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

extern template int32_t launch_i8_w<4>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<6>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<7>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<8>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<9>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<12>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<16>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_w<18>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

int32_t i8_launch_args(cudaStream_t st, const QmvCall& c, const I8Plan& p) {
    I8Args a{};
    a.wq[0] = c.wq; a.scales[0] = c.scales; a.biases[0] = c.biases;
    a.wq[1] = c.wq2; a.scales[1] = c.scales2; a.biases[1] = c.biases2;
    a.x = c.x; a.y = c.y; a.N = c.N; a.K = c.K; a.x_dtype = c.x_dtype; a.y_dtype = c.y_dtype;
    a.W = p.W; a.nblocks = p.nblocks; a.RS = p.RS; a.stg = p.stg;
    a.bs_off = p.bs_off; a.stage_off = p.stage_off;
    a.probe = g_i8_probe;
    a.fuse_norm = c.norm ? 1 : 0;
    if (c.norm) a.nf = *c.norm;
    a.status = device_status_word();
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmv: no device status word");
    const int fuse = c.wq2 ? 1 : 0;
    switch (p.J) {
        case 1: return launch_i8_w<1>(st, a, p, c.M, fuse);
        case 2: return launch_i8_w<2>(st, a, p, c.M, fuse);
        case 3: return launch_i8_w<3>(st, a, p, c.M, fuse);
        case 4: return launch_i8_w<4>(st, a, p, c.M, fuse);
        case 6: return launch_i8_w<6>(st, a, p, c.M, fuse);
        case 7: return launch_i8_w<7>(st, a, p, c.M, fuse);
        case 8: return launch_i8_w<8>(st, a, p, c.M, fuse);
        case 9: return launch_i8_w<9>(st, a, p, c.M, fuse);
        case 12: return launch_i8_w<12>(st, a, p, c.M, fuse);
        case 16: return launch_i8_w<16>(st, a, p, c.M, fuse);
        case 18: return launch_i8_w<18>(st, a, p, c.M, fuse);
    }
    return fail(LTHN_ERR_INVALID, "affine_qmv: no integer tensor-core instantiation for this plan");
}

}  // namespace lthn
