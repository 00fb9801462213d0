// Differential attention over the paged cache: every query head carries TWO score maps over the same values,
// and what leaves the head is their difference.
//
// A query head's row is [q1 | q2] (hd entries each), a key head's cache entry [k1 | k2]; values have vd entries and
// belong to the key head, not to a map.  For a row at position p, over the keys j in [from, p] of its window:
//   a_m = sum_j softmax_j((q_m . k_m,j) scale) v_j          m = 1, 2 (each map a softmax of its own)
//   o   = a_1 - lambda a_2
//   out = o / sqrt(mean(o^2) + eps) * out_scale             (a norm over the head's vd entries, no weight)
// lambda is one number for the layer and out_scale a constant (the caller's 1 - lambda_init).  Head h reads key head
// h / (heads / kv_heads).  Scores, both softmaxes, the difference and the norm are float32 whatever the storage.
//
// One block per (row, head): any sizes up to 256, float32 or bfloat16 storage; it serves prompt portions and single
// tokens alike.  The keys are cut into chunks of 32 counted from `from`, a lane a key, the block's warps taking chunks
// in turn; how a row's keys are cut depends on the row's own range only, never on what else is in the batch.
#include "common.cuh"

using namespace cj;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;
constexpr int DPL = MAX_D / 32;

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32) diff_attention_kernel(
    const TQ* __restrict__ q, TO* __restrict__ out, const TC* __restrict__ kplane, const TC* __restrict__ vplane,
    const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table, int table_stride,
    int page_tokens, int n_heads, int n_kv, int hd, int vd, int window, float scale, float lambda, float eps, float out_scale) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ float smem[];
    float* qs = smem;                         // [2 hd]
    float* acc_s = qs + 2 * hd;               // [2][WARPS][vd]
    float* ml_s = acc_s + 2 * WARPS * vd;     // [2][WARPS][2]
    float* red = ml_s + 4 * WARPS;            // [WARPS]

    const int h = blockIdx.y, t = blockIdx.x;
    const int kvh = h / (n_heads / n_kv);
    const int p = positions[t];
    const int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int* tab = table + (size_t)row_req[t] * table_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kd = 2 * hd;

    const TQ* qrow = q + ((size_t)t * n_heads + h) * kd;
    for (int d = threadIdx.x; d < kd; d += blockDim.x) qs[d] = to_f32(qrow[d]);
    __syncthreads();

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[2][DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[0][i] = acc[1][i] = 0.0f;

    const int n_chunks = (p - from + 1 + 31) / 32;
    for (int c = warp; c < n_chunks; c += WARPS) {
        const int key = from + c * 32 + lane;
        const bool valid = key <= p;
        float s[2] = {-INFINITY, -INFINITY};
        size_t base = 0;
        if (valid) {
            const int page = tab[key / page_tokens];
            base = ((size_t)page * n_kv + kvh) * page_tokens + key % page_tokens;
            const TC* kr = kplane + base * kd;
            float d0 = 0.0f, d1 = 0.0f;
            for (int d = 0; d < hd; ++d) {
                d0 = fmaf(qs[d], to_f32(kr[d]), d0);
                d1 = fmaf(qs[hd + d], to_f32(kr[hd + d]), d1);
            }
            s[0] = d0 * scale;
            s[1] = d1 * scale;
        }
        float e[2];
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
            const float m_new = fmaxf(m[mp], warp_max(s[mp]));
            const float corr = expf(m[mp] - m_new);           // 0 on the first chunk
            e[mp] = valid ? expf(s[mp] - m_new) : 0.0f;
            l[mp] = l[mp] * corr + warp_sum(e[mp]);
            m[mp] = m_new;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[mp][i] *= corr;
        }
        const int in_chunk = min(32, p - (from + c * 32) + 1);
        for (int j = 0; j < in_chunk; ++j) {
            const float e0 = __shfl_sync(0xffffffffu, e[0], j), e1 = __shfl_sync(0xffffffffu, e[1], j);
            const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
            const TC* vr = vplane + bj * vd;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) {
                    const float v = to_f32(vr[d]);
                    acc[0][i] = fmaf(e0, v, acc[0][i]);
                    acc[1][i] = fmaf(e1, v, acc[1][i]);
                }
            }
        }
    }
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        if (lane == 0) { ml_s[(mp * WARPS + warp) * 2] = m[mp]; ml_s[(mp * WARPS + warp) * 2 + 1] = l[mp]; }
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < vd) acc_s[(mp * WARPS + warp) * vd + d] = acc[mp][i];
        }
    }
    __syncthreads();
    // the warps' shares of each map put together, then the difference and its norm
    float f[2][WARPS], inv[2];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, ml_s[(mp * WARPS + w) * 2]);
        float ls = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = ml_s[(mp * WARPS + w) * 2];
            f[mp][w] = mw == -INFINITY ? 0.0f : expf(mw - mx);
            ls += ml_s[(mp * WARPS + w) * 2 + 1] * f[mp][w];
        }
        inv[mp] = 1.0f / ls;
    }
    float o[(MAX_D + WARPS * 32 - 1) / (WARPS * 32)];
    float ss = 0.0f;
    int n = 0;
    for (int d = threadIdx.x; d < vd; d += blockDim.x, ++n) {
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            a0 += acc_s[w * vd + d] * f[0][w];
            a1 += acc_s[(WARPS + w) * vd + d] * f[1][w];
        }
        const float v = a0 * inv[0] - lambda * (a1 * inv[1]);
        o[n] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) total += red[w];
    const float norm = out_scale / sqrtf(total / (float)vd + eps);
    TO* orow = out + ((size_t)t * n_heads + h) * vd;
    n = 0;
    for (int d = threadIdx.x; d < vd; d += blockDim.x, ++n) orow[d] = from_f32<TO>(o[n] * norm);
}

}  // namespace

// q [T, n_heads, 2 hd], out [T, n_heads, vd] in the activation dtype; k plane [pages, n_kv, page_tokens, 2 hd],
// v plane [pages, n_kv, page_tokens, vd].  hd: the size of ONE map's query / key.
CJ_EXPORT int cj_diff_attention(const void* q, void* out, int act_dtype, const void* kplane, const void* vplane, int cache_dtype,
                                const int* positions, const int* row_req, const int* table, int table_stride, int page_tokens,
                                int T, int n_heads, int n_kv, int hd, int vd, int window, float scale, float lambda, float eps,
                                float out_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table) return CJ_ERR_ARG;
    if (hd <= 0 || hd > MAX_D || vd <= 0 || vd > MAX_D || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0)
        return CJ_ERR_SIZE;
    if (n_heads > 65535) return CJ_ERR_SIZE;
    dim3 grid(T, n_heads);
    const size_t smem = (size_t)(2 * hd + 2 * WARPS * vd + 4 * WARPS + WARPS) * sizeof(float);
#define LAUNCH(TQ, TC)                                                                                                 \
    cj::launch(diff_attention_kernel<TQ, TC, TQ>, dim3(grid), dim3(WARPS * 32), smem, stream, (const TQ*)q, (TQ*)out,    \
               (const TC*)kplane, (const TC*)vplane, positions, row_req, table, table_stride, page_tokens, n_heads, n_kv, hd, \
               vd, window, scale, lambda, eps, out_scale)
    if (act_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (act_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}
