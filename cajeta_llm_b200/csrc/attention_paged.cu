// General paged attention: one query row and head per block, keys and values read
// from cache pages through the request's block table.  It serves a portion of a prompt
// and a single decoded token alike (every row carries its own position), any head size
// up to 256, any group size, float32 or bfloat16 storage; all arithmetic is float32.
// Values may have another size than keys (vd), a score may be capped,
// s <- cap * tanh(s / cap), and a head's output may be multiplied by the sigmoid of a gate
// value of its own (one float32 per row and head).
//
// For head h, kv head = h / (heads / kv_heads); keys t in [from, p] with
// from = p + 1 - w when w > 0 and p + 1 > w, else 0; s_t = (q . k_t) * scale; softmax
// with the maximum subtracted; o = (sum_t e_t v_t) / sum_t e_t
// (model/PagedKvCache.cajeta:374-470).  The keys of a row are cut into chunks of 32 that
// the block's warps take in turn, each keeping a running (max, sum, accumulator) as the
// reference's flash kernels do (model/AttnKernel.cajeta:883); the cut depends only on
// the row's own [from, p], so the result does not depend on the rest of the batch.
#define CJ_LIB "attention_paged"
#include "common.cuh"

using namespace cj;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;
constexpr int DPL = MAX_HD / 32;   // output dims per lane

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_kernel(
    const TQ* __restrict__ q, TO* __restrict__ out, const TC* __restrict__ kplane, const TC* __restrict__ vplane,
    const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table,
    int table_stride, int page_tokens, int n_heads, int n_kv, int hd, int vd, int window, float scale, float softcap,
    const float* __restrict__ head_gate, int gate_ld) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ float smem[];
    float* qs = smem;                       // [hd]
    float* acc_s = smem + hd;               // [WARPS][vd]
    float* m_s = acc_s + WARPS * vd;        // [WARPS]
    float* l_s = m_s + WARPS;               // [WARPS]

    int h = blockIdx.y, t = blockIdx.x;
    int kvh = h / (n_heads / n_kv);
    int p = positions[t];
    int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int* tab = table + (size_t)row_req[t] * table_stride;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const TQ* qrow = q + ((size_t)t * n_heads + h) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = to_f32(qrow[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;

    int n_keys = p - from + 1;
    int n_chunks = (n_keys + 31) / 32;
    for (int c = warp; c < n_chunks; c += WARPS) {
        int key = from + c * 32 + lane;
        bool valid = key <= p;
        float s = -INFINITY;
        size_t base = 0;                    // the key's place in units of one (token, head) entry
        if (valid) {
            int page = tab[key / page_tokens];
            base = ((size_t)page * n_kv + kvh) * page_tokens + key % page_tokens;
            const TC* kr = kplane + base * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
            s = dot * scale;
            if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
        }
        float cmax = warp_max(s);
        float m_new = fmaxf(m, cmax);
        float corr = expf(m - m_new);       // m = -inf on the first chunk: exp(-inf) = 0
        float e = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(e);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        int in_chunk = min(32, p - (from + c * 32) + 1);
        for (int j = 0; j < in_chunk; ++j) {
            float ej = __shfl_sync(0xffffffffu, e, j);
            size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
            const TC* vr = vplane + bj * vd;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                int d = lane + 32 * i;
                if (d < vd) acc[i] = fmaf(ej, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }

    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        int d = lane + 32 * i;
        if (d < vd) acc_s[warp * vd + d] = acc[i];
    }
    __syncthreads();
    float mx = m_s[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, m_s[w]);
    float f[WARPS];
    float lsum = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - mx);
        lsum += l_s[w] * f[w];
    }
    float inv = 1.0f / lsum;
    if (head_gate) inv *= 1.0f / (1.0f + expf(-head_gate[(size_t)t * gate_ld + h]));
    TO* orow = out + ((size_t)t * n_heads + h) * vd;
    for (int d = threadIdx.x; d < vd; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) o += acc_s[w * vd + d] * f[w];
        orow[d] = from_f32<TO>(o * inv);
    }
}

// ---------------------------------------------------------------------------------
// Attention whose heads talk to each other before the softmax, with a sink: one block per row, all heads.
//   raw_g,j   = (q_g . k_j) * scale * temp[g]                       (temp: a number per head, or none)
//   s_h,j     = sum_g talk[h, g] raw_g,j                            (talk: [heads, heads], or none = identity)
//   o_h       = sum_j e^(s_h,j - m) v_j / (sum_j e^(s_h,j - m) + e^(sink_h - m))   (sink: per head, or none)
// over the keys j in [from, p] of the row's window.  The sink is one more term e^(sink_h) of the
// divisor alone: sink_h is used as stored, nothing is added to the numerator.  The keys are walked in chunks of 32 from `from`
// on, the cut depending on the row's own range only: a warp takes heads in turn (lane = key) for the raw
// scores, the block meets, then a warp mixes and sums for its heads with a running maximum that starts at
// the sink.  All arithmetic is float32.
// ---------------------------------------------------------------------------------
constexpr int MIX_WARPS = 8;

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(MIX_WARPS * 32) mixed_heads_attention_kernel(
    const TQ* __restrict__ q, TO* __restrict__ out, const TC* __restrict__ kplane, const TC* __restrict__ vplane,
    const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table,
    int table_stride, int page_tokens, int n_heads, int n_kv, int hd, int vd, int window, float scale,
    const float* __restrict__ temp, const float* __restrict__ talk, const float* __restrict__ sink) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ float smem[];
    float* qs = smem;                               // [n_heads][hd]
    float* raw = qs + (size_t)n_heads * hd;         // [n_heads][32]
    float* tk = raw + (size_t)n_heads * 32;         // [n_heads][n_heads] (identity when talk is null)
    float* acc_s = tk + (size_t)n_heads * n_heads;  // [n_heads][vd]
    float* ml = acc_s + (size_t)n_heads * vd;       // [n_heads][2]: running maximum, running sum
    __shared__ unsigned long long place[32];        // the chunk's keys' places in units of one (token, kv head 0) entry

    const int t = blockIdx.x;
    const int p = positions[t];
    const int from = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int* tab = table + (size_t)row_req[t] * table_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_kv = n_heads / n_kv;

    const TQ* qrow = q + (size_t)t * n_heads * hd;
    for (int d = threadIdx.x; d < n_heads * hd; d += blockDim.x) qs[d] = to_f32(qrow[d]);
    for (int i = threadIdx.x; i < n_heads * n_heads; i += blockDim.x)
        tk[i] = talk ? talk[i] : ((i / n_heads) == (i % n_heads) ? 1.0f : 0.0f);
    for (int i = threadIdx.x; i < n_heads * vd; i += blockDim.x) acc_s[i] = 0.0f;
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        ml[2 * h] = sink ? sink[h] : -INFINITY;
        ml[2 * h + 1] = sink ? 1.0f : 0.0f;
    }
    __syncthreads();

    const int n_keys = p - from + 1;
    const int n_chunks = (n_keys + 31) / 32;
    for (int c = 0; c < n_chunks; ++c) {
        const int key0 = from + c * 32;
        const int in_chunk = min(32, p - key0 + 1);
        if (warp == 0) {
            unsigned long long b = 0;
            if (lane < in_chunk) {
                const int key = key0 + lane;
                const int page = tab[key / page_tokens];
                b = (unsigned long long)page * n_kv * page_tokens + key % page_tokens;
            }
            place[lane] = b;
        }
        __syncthreads();
        // raw scores: a warp a head, a lane a key
        for (int g = warp; g < n_heads; g += MIX_WARPS) {
            float s = 0.0f;
            if (lane < in_chunk) {
                const TC* kr = kplane + (place[lane] + (size_t)(g / per_kv) * page_tokens) * hd;
                const float* qh = qs + (size_t)g * hd;
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qh[d], to_f32(kr[d]), dot);
                s = dot * scale;
                if (temp) s *= temp[g];
            }
            raw[g * 32 + lane] = s;
        }
        __syncthreads();
        // mixing, running softmax and weighted values: a warp a head
        for (int h = warp; h < n_heads; h += MIX_WARPS) {
            float s = 0.0f;
            for (int g = 0; g < n_heads; ++g) s = fmaf(tk[h * n_heads + g], raw[g * 32 + lane], s);
            if (lane >= in_chunk) s = -INFINITY;
            const float m = ml[2 * h], l = ml[2 * h + 1];
            const float m_new = fmaxf(m, warp_max(s));
            const float corr = expf(m - m_new);             // m = -inf before the first key without a sink: 0
            const float e = lane < in_chunk ? expf(s - m_new) : 0.0f;
            const float l_new = l * corr + warp_sum(e);
            const size_t kv_off = (size_t)(h / per_kv) * page_tokens;
            for (int d0 = 0; d0 < vd; d0 += 32) {
                const int d = d0 + lane;
                float a = d < vd ? acc_s[(size_t)h * vd + d] * corr : 0.0f;
                for (int j = 0; j < in_chunk; ++j) {
                    const float ej = __shfl_sync(0xffffffffu, e, j);
                    if (d < vd) a = fmaf(ej, to_f32(vplane[(place[j] + kv_off) * vd + d]), a);
                }
                if (d < vd) acc_s[(size_t)h * vd + d] = a;
            }
            __syncwarp();
            if (lane == 0) { ml[2 * h] = m_new; ml[2 * h + 1] = l_new; }
            __syncwarp();
        }
        __syncthreads();
    }
    TO* orow = out + (size_t)t * n_heads * vd;
    for (int i = threadIdx.x; i < n_heads * vd; i += blockDim.x) orow[i] = from_f32<TO>(acc_s[i] / ml[2 * (i / vd) + 1]);
}

}  // namespace

// q [T, n_heads, hd], out [T, n_heads, vd] in the activation dtype; planes [pages, n_kv, page_tokens, hd | vd].
// temp [n_heads], talk [n_heads, n_heads] (row h = the weights of head h's mixed score), sink [n_heads]: float32 or null.
CJ_EXPORT int cj_mixed_heads_attention(const void* q, void* out, int act_dtype, const void* kplane, const void* vplane,
                                       int cache_dtype, const int* positions, const int* row_req, const int* table,
                                       int table_stride, int page_tokens, int T, int n_heads, int n_kv, int hd, int vd,
                                       int window, float scale, const float* temp, const float* talk, const float* sink,
                                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table) return CJ_ERR_ARG;
    if (hd <= 0 || vd <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    const size_t smem = ((size_t)n_heads * (hd + 32 + n_heads + vd + 2)) * sizeof(float);
    if (smem > 200 * 1024) return CJ_ERR_SIZE;
#define LAUNCH(TQ, TC)                                                                                                  \
    do {                                                                                                                \
        static size_t sized = 48 * 1024;                                                                                \
        if (smem > sized) {                                                                                             \
            cudaFuncSetAttribute(mixed_heads_attention_kernel<TQ, TC, TQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            sized = smem;                                                                                               \
        }                                                                                                               \
        cj::launch(mixed_heads_attention_kernel<TQ, TC, TQ>, dim3(T), dim3(MIX_WARPS * 32), smem, stream, (const TQ*)q, (TQ*)out, \
            (const TC*)kplane, (const TC*)vplane, positions, row_req, table, table_stride, page_tokens, n_heads, n_kv, hd, vd, \
            window, scale, temp, talk, sink);                                                                           \
    } while (0)
    if (act_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (act_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}

// q [T, n_heads, hd], out [T, n_heads, vd] in the activation dtype; planes [pages, n_kv, page_tokens, hd | vd].
// softcap 0: none.  head_gate: null, or float32 with row stride gate_ld whose entry [t, h] gates head h of row t.
CJ_EXPORT int cj_paged_attention(const void* q, void* out, int act_dtype, const void* kplane, const void* vplane,
                                 int cache_dtype, const int* positions, const int* row_req, const int* table,
                                 int table_stride, int page_tokens, int T, int n_heads, int n_kv, int hd, int vd,
                                 int window, float scale, float softcap, const float* head_gate, int gate_ld,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !row_req || !table) return CJ_ERR_ARG;
    if (vd <= 0 || vd > MAX_HD) return CJ_ERR_SIZE;
    if (hd <= 0 || hd > MAX_HD || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (n_heads > 65535) return CJ_ERR_SIZE;
    dim3 grid(T, n_heads);
    size_t smem = (size_t)(hd + WARPS * vd + 2 * WARPS) * sizeof(float);
#define LAUNCH(TQ, TC)                                                                                             \
    cj::launch(paged_attention_kernel<TQ, TC, TQ>, dim3(grid), dim3(WARPS * 32), smem, stream, (const TQ*)q, (TQ*)out, (const TC*)kplane, \
        (const TC*)vplane, positions, row_req, table, table_stride, page_tokens, n_heads, n_kv, hd, vd, window, scale, softcap, \
        head_gate, gate_ld)
    if (act_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (act_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}

// ---------------------------------------------------------------------------------
// Heads of a step's rows made ready for attention, one warp per (row, head): the
// queries' and keys' heads are RMS-normed over the head (x / sqrt(mean x^2 + eps) * w[d],
// one weight vector shared by the heads) when a weight is given; their first `rot` entries
// are rotated at the row's position, entry i paired with entry i + rot/2:
//   (a, b) -> (a cos - b sin, b cos + a sin), angle = float(p) * inv_freq[i],
// cos and sin multiplied by `magnitude`; queries go to q_out, keys and values to the row's
// place in the paged cache.  v_off < 0: the values are the keys as projected, before norm
// and rotation (vd == hd then).  All arithmetic is float32.
// `q_temp_coef` != 0: the queries (not the keys) are multiplied by 1 + coef ln(floor((p + 1) / every) + 1), a temperature
// that grows with the row's position p in steps of `every` tokens.
// `whole`: the norm's statistic is taken over all heads of q (of k) at once, mean over n_heads * hd
// (n_kv * hd) entries, and the weight has that many entries, a head reading its own stretch.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void store4(float* dst, float4 v) { *(float4*)dst = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *(unsigned*)&lo;
    u.y = *(unsigned*)&hi;
    *(uint2*)dst = u;
}
__device__ __forceinline__ float4 mul4(float4 a, float f) { return make_float4(a.x * f, a.y * f, a.z * f, a.w * f); }
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }

// One block per row (with few rows the row's heads are shared out over gridDim.y blocks): the row's cos
// and sin are worked out once into shared memory, then a warp takes a head at a time.  Head sizes, rotary
// parts and offsets that are multiples of four go four entries a lane (16-byte loads, 8- or 16-byte stores).
template <typename TQ, typename TC>
__global__ void __launch_bounds__(128) head_prepare_kernel(
    const float* __restrict__ x, int ld, int q_off, int k_off, int v_off, TQ* __restrict__ q_out, TC* __restrict__ kplane,
    TC* __restrict__ vplane, const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table,
    int table_stride, int page_tokens, int T, int n_heads, int n_kv, int hd, int vd, int rot, const float* __restrict__ inv_freq,
    float magnitude, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, int write_kv, int whole,
    float q_temp_coef, int q_temp_every) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(16) float cs[];      // cos[half] then sin[half], times the magnitude
    __shared__ float whole_sum[2][4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot >> 1;
    // a query's temperature grows with its position in steps of `every` tokens: 1 + coef ln(floor((p + 1) / every) + 1)
    const float q_temp = q_temp_coef != 0.0f ? 1.0f + q_temp_coef * logf((float)((pos + 1) / q_temp_every) + 1.0f) : 1.0f;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[i] = cosf(ang) * magnitude;
        cs[half + i] = sinf(ang) * magnitude;
    }
    size_t place0 = 0;
    bool have_page = false;
    if (write_kv) {
        const int page = table[(size_t)row_req[t] * table_stride + pos / page_tokens];
        have_page = page >= 0;                       // no page: the host never schedules this
        place0 = (size_t)(have_page ? page : 0) * n_kv * page_tokens + pos % page_tokens;
    }
    const float* xrow = x + (size_t)t * ld;
    float inv_whole[2] = {1.0f, 1.0f};
    if (whole) {
        // every block of the row sums the whole of q and of k in the same order: the same bits in each
        float sq = 0.0f, sk = 0.0f;
        if (q_norm) for (int d = threadIdx.x; d < n_heads * hd; d += blockDim.x) sq = fmaf(xrow[q_off + d], xrow[q_off + d], sq);
        if (k_norm && write_kv) for (int d = threadIdx.x; d < n_kv * hd; d += blockDim.x) sk = fmaf(xrow[k_off + d], xrow[k_off + d], sk);
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { whole_sum[0][warp] = sq; whole_sum[1][warp] = sk; }
    }
    __syncthreads();
    if (whole) {
        const float sq = whole_sum[0][0] + whole_sum[0][1] + whole_sum[0][2] + whole_sum[0][3];
        const float sk = whole_sum[1][0] + whole_sum[1][1] + whole_sum[1][2] + whole_sum[1][3];
        inv_whole[0] = 1.0f / sqrtf(sq / (float)(n_heads * hd) + eps);
        inv_whole[1] = 1.0f / sqrtf(sk / (float)(n_kv > 0 ? n_kv * hd : 1) + eps);
    }
    const int slots = n_heads + (write_kv && have_page ? n_kv : 0);
    const bool vec = (hd % 4 == 0) && hd <= 256 && (half % 4 == 0) && (vd % 4 == 0) && ((ld | q_off | k_off | (v_off < 0 ? 0 : v_off)) % 4 == 0) &&
                     ((((uintptr_t)x) | ((uintptr_t)q_out) | ((uintptr_t)kplane) | ((uintptr_t)vplane) | ((uintptr_t)q_norm) |
                       ((uintptr_t)k_norm)) & 15) == 0;
    for (int slot = blockIdx.y * 4 + warp; slot < slots; slot += gridDim.y * 4) {
        const bool is_q = slot < n_heads;
        const int head = is_q ? slot : slot - n_heads;
        const float* src = xrow + (is_q ? q_off : k_off) + head * hd;
        const float* nw = is_q ? q_norm : k_norm;
        if (nw && whole) nw += (size_t)head * hd;
        const size_t place = place0 + (size_t)head * page_tokens;
        float inv = 1.0f;
        // the four-a-lane form keeps the head's entries (at most 256: two groups of four a lane) in registers
        // between the sum of squares and the rotation
        float4 held[2];
        if (vec) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int d = lane * 4 + k * 128;
                held[k] = d < hd ? *(const float4*)(src + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        if (nw && whole) {
            inv = inv_whole[is_q ? 0 : 1];
        } else if (nw) {
            float ss = 0.0f;
            if (vec) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float4 a = held[k];
                    ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
                }
            } else {
                for (int d = lane; d < hd; d += 32) ss = fmaf(src[d], src[d], ss);
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        if (is_q) inv *= q_temp;
        if (vec) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int d = lane * 4 + k * 128;
                if (d >= hd) break;
                float4 a = mul4(held[k], inv);
                if (nw) a = mul4(a, *(const float4*)(nw + d));
                if (d < rot) {
                    const bool low = d < half;
                    const int i = low ? d : d - half, pd = low ? d + half : d - half;
                    float4 b = mul4(*(const float4*)(src + pd), inv);
                    if (nw) b = mul4(b, *(const float4*)(nw + pd));
                    const float4 c = *(const float4*)(cs + i), sn = *(const float4*)(cs + half + i);
                    const float sg = low ? -1.0f : 1.0f;
                    a = make_float4(fmaf(sg * b.x, sn.x, a.x * c.x), fmaf(sg * b.y, sn.y, a.y * c.y), fmaf(sg * b.z, sn.z, a.z * c.z),
                                    fmaf(sg * b.w, sn.w, a.w * c.w));
                }
                if (is_q) store4(q_out + ((size_t)t * n_heads + head) * hd + d, a);
                else store4(kplane + place * hd + d, a);
            }
            if (!is_q) {
                const float* vs = v_off < 0 ? src : xrow + v_off + head * vd;
                for (int d = lane * 4; d < vd; d += 128) store4(vplane + place * vd + d, *(const float4*)(vs + d));
            }
            continue;
        }
        for (int d = lane; d < hd; d += 32) {
            float a = src[d] * inv * (nw ? nw[d] : 1.0f);
            float r = a;
            if (d < rot) {
                const int i = d < half ? d : d - half, pd = d < half ? d + half : d - half;
                const float b = src[pd] * inv * (nw ? nw[pd] : 1.0f);
                r = d < half ? a * cs[i] - b * cs[half + i] : a * cs[i] + b * cs[half + i];
            }
            if (is_q) q_out[((size_t)t * n_heads + head) * hd + d] = from_f32<TQ>(r);
            else kplane[place * hd + d] = from_f32<TC>(r);
        }
        if (!is_q) {
            const float* vs = v_off < 0 ? src : xrow + v_off + head * vd;
            for (int d = lane; d < vd; d += 32) vplane[place * vd + d] = from_f32<TC>(vs[d]);
        }
    }
}

CJ_EXPORT int cj_head_prepare(const float* x, int ld, int q_off, int k_off, int v_off, void* q_out, int q_dtype, void* kplane,
                              void* vplane, int cache_dtype, const int* positions, const int* row_req, const int* table,
                              int table_stride, int page_tokens, int T, int n_heads, int n_kv, int hd, int vd, int rotary_dim,
                              const float* inv_freq, float magnitude, const float* q_norm, const float* k_norm, float eps,
                              int write_kv, int whole, float q_temp_coef, int q_temp_every, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!x || !q_out || !positions || n_heads <= 0 || hd <= 0 || vd <= 0) return CJ_ERR_ARG;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return CJ_ERR_SIZE;
    if (rotary_dim > 0 && !inv_freq) return CJ_ERR_ARG;
    if (write_kv && (!kplane || !vplane || !row_req || !table || page_tokens <= 0 || n_kv <= 0)) return CJ_ERR_ARG;
    if (v_off < 0 && vd != hd) return CJ_ERR_SIZE;
    if (q_temp_coef != 0.0f && q_temp_every < 1) return CJ_ERR_SIZE;
    // a warp a head; with few rows the heads of a row go over several blocks
    const int slots = n_heads + (write_kv ? n_kv : 0);
    int parts = T >= 128 ? 1 : (slots + 3) / 4;
    if (parts > 16) parts = 16;
    dim3 grid(T, parts);
    const size_t smem = (size_t)rotary_dim * sizeof(float);
#define LAUNCH(TQ, TC)                                                                                                  \
    cj::launch(head_prepare_kernel<TQ, TC>, dim3(grid), dim3(128), smem, stream, x, ld, q_off, k_off, v_off, (TQ*)q_out,  \
        (TC*)kplane, (TC*)vplane, positions, row_req, table, table_stride, page_tokens, T, n_heads, n_kv, hd, vd,      \
        rotary_dim, inv_freq, magnitude, q_norm, k_norm, eps, write_kv, whole, q_temp_coef, q_temp_every)
    if (q_dtype == CJ_F32 && cache_dtype == CJ_F32) LAUNCH(float, float);
    else if (q_dtype == CJ_BF16 && cache_dtype == CJ_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef LAUNCH
    return launch_status();
}
