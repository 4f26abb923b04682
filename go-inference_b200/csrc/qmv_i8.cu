// qmv_i8.cu — planning and dispatch of the integer tensor-core affine_qmv kernel
// (kernel and its description: qmv_i8_kernel.cuh; instantiations: qmv_i8_inst*.cu).
#include "common.cuh"
#include "qmv.hpp"

#include <algorithm>

namespace lthn {

struct I8Args;
template <int J>
int32_t launch_i8_w(cudaStream_t st, const I8Args& a, const I8Plan& p, int M, int fuse);
int32_t i8_launch_args(cudaStream_t st, const QmvCall& c, const I8Plan& p);

// ---- host side --------------------------------------------------------------------

int g_i8_stg = 0, g_i8_probe = 0;  // measurement aids
static const int kI8J[] = {1, 2, 3, 4, 6, 7, 8, 9, 12, 16, 18};

bool i8_plan(int64_t N, int64_t K, int M, int fuse, int force_rt, int force_w, I8Plan* p) {
    if (M < 1 || M > 2 || K % 64 != 0 || N < 16 || N % 16 != 0) return false;
    const int G = (int)(K / 64);
    // (J, W): W consumer warps of J groups each. Measured on B200: a long stream (many row blocks
    // per SM) runs fastest with few warps per block and many blocks per SM (less hand-off per row
    // block, more independent pipelines: 5.9 TB/s with 4 warps against 4.4 with 12 on the 340 MB
    // lm_head); a small matrix, where each block sees only a few row blocks, finishes sooner with
    // the groups spread over as many warps as possible.
    const double per_sm = (double)(N / 16) / 148.0;
    const int target = per_sm < 10.0 ? 16 : (per_sm < 20.0 ? 7 : 4);
    int J = 0, W = 0, best = -1;
    for (int cand : kI8J) {
        if (G % cand) continue;
        const int w = G / cand;
        if (w < 1 || w > 16) continue;
        if (cand > 9 && w > 8) continue;  // many groups per warp only in small blocks (registers)
        int score = 1000 - 10 * std::abs(w - target) + (target >= 8 ? w : -w);
        if (force_w > 0) score = (w == force_w) ? 5000 : -1;
        if (score > best) { best = score; J = cand; W = w; }
    }
    if (best < 0) return false;
    const int sets = fuse ? 2 : 1;
    const int rsw = (int)(K / 8);
    const int padw = ((8 - rsw % 32) + 32) % 32;
    const int RS = (rsw + padw) * 4;
    (void)force_rt;
    for (int RT = 1; RT >= 1; RT--) {
        const int RB = 16 * RT;
        const int nblocks = (int)((N + RB - 1) / RB);
        const size_t sb = ((size_t)RB * G * 2 + 15) / 16 * 16;
        const size_t stage = sets * ((size_t)RB * RS + 2 * sb);
        for (int stg = g_i8_stg >= 2 && g_i8_stg <= 4 ? g_i8_stg : 2; stg >= 2; stg--) {
            const size_t part_bytes = (size_t)2 * stg * W * sets * RB * M * 4;
            const size_t bs_off = 512 + part_bytes;
            const size_t stage_off = (bs_off + (size_t)W * M * 192 + 127) / 128 * 128;
            const size_t smem = stage_off + (size_t)stg * stage;
            if (smem > 200 * 1024) continue;
            p->J = J; p->W = W; p->RT = RT; p->stg = stg; p->RS = RS; p->nblocks = nblocks;
            p->threads = (W + 1) * 32;
            p->bs_off = (int)bs_off; p->stage_off = (int)stage_off;
            p->smem = smem;
            return true;
        }
    }
    return false;
}

bool qmv_can_fuse_norm(int64_t N, int64_t K, int M, bool geglu) {
    I8Plan p;
    return i8_plan(N, K, M, geglu ? 1 : 0, 0, 0, &p);
}

int32_t i8_launch(cudaStream_t st, const QmvCall& c, const I8Plan& p) { return i8_launch_args(st, c, p); }

}  // namespace lthn
