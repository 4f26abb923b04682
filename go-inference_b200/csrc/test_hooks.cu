// test_hooks.cu — entry points that exist only in the test build of the library
// (liblthn_cuda_hooks.so = the product's objects + this file). They override kernel
// dispatch so that every kernel variant can be driven through the C ABI, and run the
// tensor-parallel norm on one GPU. The product library exports none of them, and the
// variables they set are not visible outside the shared object.
#include "common.cuh"
#include "decoder_kernels.hpp"
#include "qmv.hpp"

namespace lthn {
extern LTHN_HIDDEN int g_force_rt, g_force_warps, g_force_kernel;  // qmv.cu
extern LTHN_HIDDEN int g_force_nt;                                 // qmm.cu
}  // namespace lthn

using namespace lthn;

extern "C" {

// rt: rows per thread (dp4a) / 16-row tiles per CTA (bf16 tensor-core kernel) / K slices (integer
// kernel); nwarps: warps per CTA. 0 restores the defaults.
void lthn_debug_qmv_force_config(int32_t rt, int32_t nwarps) {
    g_force_rt = rt;
    g_force_warps = nwarps;
}
// kernel: 0 default dispatch, 1 dp4a, 2 bf16 mma.sync, 3 integer tensor-core, 4 tcgen05 streaming; bits 8-10: ring stages of the
// integer kernel (0 default)
void lthn_debug_qmv_force_kernel(int32_t kernel) {
    g_force_kernel = kernel & 15;
    g_i8_stg = (kernel >> 8) & 7;
}
void lthn_debug_qmm_force_tile(int32_t nt) { g_force_nt = nt; }

// The plan the integer tensor-core matvec would run for a call (host logic only, no CUDA call): returns 1 and
// out = {J, W, stg, RS, nblocks, threads, bs_off, stage_off, ks, Gs, fuse, smem bytes}, or 0 when the kernel
// does not serve the shape. bits 4 or 8; fuse: a GeGLU pair; norm: a fused norm prologue; slices: the most K
// slices the 4-bit plan may use (the 8-bit plan slices by itself).
int32_t lthn_debug_i8_plan(int64_t N, int64_t K, int32_t M, int32_t bits, int32_t fuse, int32_t norm, int32_t slices, int64_t* out) {
    I8Plan p{};
    const bool ok = bits == 8 ? i8_plan_b8(N, K, M, &p, 0, 0, fuse, norm != 0)
                              : i8_plan(N, K, M, fuse, 0, 0, &p, slices > 1 ? slices : 1, norm != 0);
    if (!ok) return 0;
    const int64_t v[12] = {p.J, p.W, p.stg, p.RS, p.nblocks, p.threads, p.bs_off, p.stage_off, p.ks, p.Gs, p.fuse, (int64_t)p.smem};
    for (int i = 0; i < 12; i++) out[i] = v[i];
    return 1;
}

// The tensor-parallel residual norm on one GPU: the t "ranks" are t local buffers ([t][rows*width]
// in parts). flags_preset != 0: every "peer" has already signalled, nothing waits, and the call
// checks the rank-order sum and the fused norms. flags_preset == 0: no peer ever signals, so the
// bounded wait of the kernel runs out after poll_limit polls, the kernel records it and returns
// by itself, and the call reports LTHN_ERR_DEVICE_WAIT. scratch: at least 512 bytes of device memory.
int32_t lthn_debug_rmsnorm_gather_local(void* stream, const float* parts, int32_t t, void* scratch, float* h,
                                        const float* w_post, const float* w_next, float* out, int32_t rows,
                                        int32_t width, float eps, int32_t flags_preset, uint32_t poll_limit) {
    clear_error();
    LTHN_REQUIRE(parts && scratch && h && w_post && w_next && out && rows > 0 && width > 0 && t >= 2 && t <= 8,
                 "lthn_debug_rmsnorm_gather_local: bad arguments");
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t init[128] = {};
    if (flags_preset)
        for (int r = 0; r < 8; r++) init[r] = 1u;  // every "peer" already signalled exchange 1
    LTHN_CUDA_TRY(cudaMemcpyAsync(scratch, init, sizeof(init), cudaMemcpyHostToDevice, s));
    LTHN_CUDA_TRY(cudaStreamSynchronize(s));
    PeerGather g{};
    g.t = t; g.rank = 0;
    g.flag_in = (const uint32_t*)scratch;
    g.ctr = (uint32_t*)scratch + 64;
    g.status = device_status_word();
    g.poll_limit = poll_limit;
    if (!g.status) return fail(LTHN_ERR_CUDA, "no device status word");
    for (int r = 0; r < t; r++) {
        g.part[r] = parts + (size_t)r * rows * width;
        g.flag_out[r] = (uint32_t*)scratch + 16;  // a dummy line: CTA 0 writes its own signal there
    }
    int32_t rc = launch_rmsnorm_gather(s, g, h, w_post, w_next, out, rows, width, eps, nullptr, 0);
    if (rc) return rc;
    return check_device_status(s);
}

}  // extern "C"
