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
extern template int32_t launch_i8_w<21>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<2>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<3>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<4>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<6>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<9>(cudaStream_t, const I8Args&, const I8Plan&, int, int);
extern template int32_t launch_i8_b8<12>(cudaStream_t, const I8Args&, const I8Plan&, int, int);

// y[i] = sum over the K slices of part[s][i], slices added in order
__global__ void sum_parts_kernel(const float* __restrict__ part, int ks, int64_t n, void* __restrict__ y, int y_dtype) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = part[i];
    for (int s = 1; s < ks; s++) v += part[(int64_t)s * n + i];
    if (y_dtype == LTHN_DTYPE_BF16) ((uint16_t*)y)[i] = f32_to_bf16_bits(v);
    else ((float*)y)[i] = v;
}

int32_t launch_sum_parts(cudaStream_t st, const float* part, int ks, int64_t n, void* y, int y_dtype) {
    LTHN_CUDA_TRY(launch_k(sum_parts_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, part, ks, n, y, y_dtype));
    return LTHN_OK;
}

int32_t i8_launch_args(cudaStream_t st, const QmvCall& c, const I8Plan& p) {
    I8Args a{};
    a.wq[0] = c.wq; a.scales[0] = c.scales; a.biases[0] = c.biases;
    a.wq[1] = c.wq2; a.scales[1] = c.scales2; a.biases[1] = c.biases2;
    a.x = c.x; a.y = c.y; a.N = c.N; a.K = c.K; a.x_dtype = c.x_dtype; a.y_dtype = c.y_dtype;
    a.W = p.W; a.nblocks = p.nblocks; a.RS = p.RS; a.stg = p.stg;
    a.bs_off = p.bs_off; a.stage_off = p.stage_off;
    a.fuse_norm = c.norm ? 1 : 0;
    if (c.norm) { a.nf = *c.norm; a.nf.inv_width = 1.0 / (double)c.K; }
    a.npush = c.npush;
    a.push = c.push;
    if (c.npush && (c.y_dtype != LTHN_DTYPE_F32 || p.ks != 1 || c.wq2)) return fail(LTHN_ERR_INVALID, "affine_qmv: pushed results are f32, whole rows, no GeGLU");
    a.ks = p.ks; a.Gs = p.Gs;
    a.bits = c.bits;
    if (c.bits == 8 && c.npush) return fail(LTHN_ERR_INVALID, "affine_qmv: 8-bit codes do not push their results to peers");
    if (c.norm && p.ks != 1) return fail(LTHN_ERR_INVALID, "affine_qmv: a fused norm prologue needs whole rows");
    if (p.ks > 1) {
        if (c.parts) {
            a.ypart = c.parts;
        } else {
            void* ws = nullptr;
            int32_t rc = scratch_get((size_t)p.ks * c.M * c.N * sizeof(float), &ws, 4);
            if (rc) return rc;
            a.ypart = (float*)ws;
        }
    } else if (c.parts) {
        a.y = c.parts;  // a single "partial": the result itself, f32
        a.y_dtype = LTHN_DTYPE_F32;
    }
    if (c.nparts) *c.nparts = p.ks;
    a.status = device_status_word();
    if (!a.status) return fail(LTHN_ERR_CUDA, "affine_qmv: no device status word");
    const int fuse = c.wq2 ? p.fuse : 0;  // 1: two full sets per row block, 2: interleaved
    int32_t rc = LTHN_ERR_INVALID;
    if (c.bits == 8) {
        switch (p.J) {
            case 2: rc = launch_i8_b8<2>(st, a, p, c.M, fuse); break;
            case 3: rc = launch_i8_b8<3>(st, a, p, c.M, fuse); break;
            case 4: rc = launch_i8_b8<4>(st, a, p, c.M, fuse); break;
            case 6: rc = launch_i8_b8<6>(st, a, p, c.M, fuse); break;
            case 9: rc = launch_i8_b8<9>(st, a, p, c.M, fuse); break;
            case 12: rc = launch_i8_b8<12>(st, a, p, c.M, fuse); break;
            default: return fail(LTHN_ERR_INVALID, "affine_qmv: no 8-bit integer tensor-core instantiation for this plan");
        }
    } else
    switch (p.J) {
        case 1: rc = launch_i8_w<1>(st, a, p, c.M, fuse); break;
        case 2: rc = launch_i8_w<2>(st, a, p, c.M, fuse); break;
        case 3: rc = launch_i8_w<3>(st, a, p, c.M, fuse); break;
        case 4: rc = launch_i8_w<4>(st, a, p, c.M, fuse); break;
        case 6: rc = launch_i8_w<6>(st, a, p, c.M, fuse); break;
        case 7: rc = launch_i8_w<7>(st, a, p, c.M, fuse); break;
        case 8: rc = launch_i8_w<8>(st, a, p, c.M, fuse); break;
        case 9: rc = launch_i8_w<9>(st, a, p, c.M, fuse); break;
        case 12: rc = launch_i8_w<12>(st, a, p, c.M, fuse); break;
        case 16: rc = launch_i8_w<16>(st, a, p, c.M, fuse); break;
        case 18: rc = launch_i8_w<18>(st, a, p, c.M, fuse); break;
        case 21: rc = launch_i8_w<21>(st, a, p, c.M, fuse); break;
        default: return fail(LTHN_ERR_INVALID, "affine_qmv: no integer tensor-core instantiation for this plan");
    }
    if (rc) return rc;
    if (p.ks > 1 && !c.parts) {
        const int64_t n = (int64_t)c.M * c.N;
        LTHN_CUDA_TRY(launch_k(sum_parts_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)a.ypart, p.ks, n, c.y, c.y_dtype));
    }
    return LTHN_OK;
}

}  // namespace lthn
