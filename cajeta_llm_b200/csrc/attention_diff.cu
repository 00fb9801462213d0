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
// Two forms:
//   diff_attention_kernel   one block per (row, head): the general form, any sizes up to 256, float32 or bfloat16
//                           storage; serves prompt portions and single tokens alike.  The keys are cut into chunks of
//                           32 counted from `from`, a lane a key, the block's warps taking chunks in turn.
//   diff_flash_kernel       bfloat16 storage, a map's size 32, 64 or 128 and values of 64 or 128: 64 query rows of one
//                           request and one head per block of eight warps.  Warps 0-3 run map 1 and warps 4-7 map 2 for
//                           the same rows over the SAME tiles of keys and values in shared memory (cp.async straight from
//                           the pages, the next chunk of 64 keys in flight): scores and value products on the tensor
//                           cores (mma.sync m16n8k16, bf16 in, f32 out), the running softmax of each map in float32
//                           registers.  A weight enters the value product as two bfloat16 terms, its rounding and the
//                           rest, so the weights stay float32-grade.  At the end map 2's warps hand their normalised
//                           sums over through shared memory and map 1's warps take the difference and the norm.
//                           With few rows in the step a row block's keys are dealt to `splits` blocks in stretches
//                           of split_keys; each leaves (sum, maximum, weight sum) per map and diff_merge_kernel puts
//                           them together in stretch order, takes the difference and norms.
// In both, how a row's keys are cut depends on the row's own range (and, in the split form, on a stretch length the
// caller fixes for the step's shape), never on what else is in the batch.
#define CJ_LIB "attention_diff"
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

// ---------------------------------------------------------------------------------
// the tiled form
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two weights as bfloat16 pairs: their roundings, and what the roundings left over
__device__ __forceinline__ void split_pair(float a, float b, unsigned& hi, unsigned& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - __low2float(h), b - __high2float(h));
    hi = *(const unsigned*)&h;
    lo = *(const unsigned*)&l;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}
// element (row, col) of a [rows][D] bf16 tile whose 16-byte pieces are XOR-swizzled by row (D a multiple of 64)
template <int D>
__device__ __forceinline__ __nv_bfloat16* tile_ptr(__nv_bfloat16* base, int row, int col) {
    const int chunk = (col >> 3) ^ (row & 7);
    return base + row * D + chunk * 8 + (col & 7);
}

constexpr int BN = 64;      // keys a chunk

// partial: [splits][T][n_heads][2][DV + 2] float32 (unnormalised sums, then the maximum in units of log 2 and the weight sum)
// BM: rows a block (64 for steps with prompt portions; 16 for steps of single tokens, where a block is two warps, one a map,
// and three blocks share a SM, each with a chunk of keys in flight)
template <int HD, int DV, int BM>
__global__ void __launch_bounds__(BM * 4) diff_flash_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kplane,
    const __nv_bfloat16* __restrict__ vplane, const int* __restrict__ req_start, const int* __restrict__ req_prior,
    int n_requests, int T, const int* __restrict__ table, int table_stride, int page_tokens, int n_heads, int n_kv, int window,
    float scale_log2, float lambda, float eps, float out_scale, int split_keys, float* __restrict__ partial) {
    // launched in plain stream order (launch_in_order): everything before it has ended, and what follows starts when
    // it has ended
    constexpr int KD = 2 * HD;
    constexpr int NW = BM / 16;                                     // warps a map
    constexpr int FLASH_THREADS = 2 * NW * 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                 // [BM][KD]
    __nv_bfloat16* ks = qs + BM * KD;                             // [2][BN][KD]
    __nv_bfloat16* vs = ks + 2 * BN * KD;                         // [2][BN][DV]
    constexpr int CK = KD / 8, CV = DV / 8;

    // which request and which tile of its rows; late tiles (the most keys) start first
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, req = -1, row0 = 0, rows = 0, first = 0;
    for (int r = 0; r < n_requests; ++r) {
        const int lo = req_start[r], hi = req_start[r + 1];
        const int tiles = (hi - lo + BM - 1) / BM;
        if (tile < first + tiles) {
            req = r;
            row0 = lo + (tile - first) * BM;
            rows = min(BM, hi - row0);
            break;
        }
        first += tiles;
    }
    if (req < 0) return;
    const int h = blockIdx.y;
    const int kvh = h / (n_heads / n_kv);
    const int p0 = req_prior[req] + (row0 - req_start[req]);
    const int p_last = p0 + rows - 1;
    // the keys this block walks: the tile's range, cut to the block's stretch when the keys are dealt out
    int key_lo = (window > 0 && p0 + 1 > window) ? p0 + 1 - window : 0;
    int key_hi = p_last;
    if (split_keys > 0) {
        key_lo = max(key_lo, (int)blockIdx.z * split_keys);
        key_hi = min(key_hi, ((int)blockIdx.z + 1) * split_keys - 1);
        if ((int)blockIdx.z * split_keys > p_last) return;        // the merge never reads a stretch that starts past a row
    }
    const int kt_begin = key_lo / BN, kt_end = key_hi / BN;         // key_lo > key_hi: a window that left this stretch behind
    const int* tab = table + (size_t)req * table_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mp = warp / NW;                                       // the map this warp runs
    const int wrow = (warp % NW) * 16;

    // where the keys of a chunk lie: the row of (page, key head, place in the page) in units of one cache entry, or -1 past the
    // block's last key; worked out a chunk ahead by one thread a key, so that the copies below only read it
    __shared__ int row_at[2][BN];
    auto find_rows = [&](int kt) {
        for (int r = tid; r < BN; r += FLASH_THREADS) {
            const int key = kt * BN + r;
            row_at[kt & 1][r] = key <= p_last ? (tab[key / page_tokens] * n_kv + kvh) * page_tokens + key % page_tokens : -1;
        }
    };
    auto load_kv = [&](int kt, int buf) {
        __nv_bfloat16* kd = ks + buf * BN * KD;
        __nv_bfloat16* vd = vs + buf * BN * DV;
        const int* at = row_at[kt & 1];
        for (int i = tid; i < BN * CK; i += FLASH_THREADS) {
            const int r = i / CK, c = i % CK;
            const int row = at[r];
            cp_async16(kd + r * KD + (c ^ (r & 7)) * 8, kplane + (row < 0 ? 0 : (size_t)row * KD + c * 8), row >= 0);
        }
        for (int i = tid; i < BN * CV; i += FLASH_THREADS) {
            const int r = i / CV, c = i % CV;
            const int row = at[r];
            cp_async16(vd + r * DV + (c ^ (r & 7)) * 8, vplane + (row < 0 ? 0 : (size_t)row * DV + c * 8), row >= 0);
        }
    };
    if (kt_begin <= kt_end) find_rows(kt_begin);
    if (kt_begin < kt_end) find_rows(kt_begin + 1);
    __syncthreads();
    for (int i = tid; i < BM * CK; i += FLASH_THREADS) {
        const int r = i / CK, c = i % CK;
        const bool valid = r < rows;
        const __nv_bfloat16* src = q + ((size_t)(row0 + (valid ? r : 0)) * n_heads + h) * KD + c * 8;
        cp_async16(qs + r * KD + (c ^ (r & 7)) * 8, src, valid);
    }
    if (kt_begin <= kt_end) load_kv(kt_begin, 0);
    cp_async_commit();

    const int g = lane >> 2, t4 = lane & 3;
    float o[DV / 8][4];
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.0f, 0.0f};      // rows g and g + 8
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const int pos0 = p0 + wrow + g, pos1 = pos0 + 8;
    const int from0 = max(key_lo, (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0);
    const int from1 = max(key_lo, (window > 0 && pos1 + 1 > window) ? pos1 + 1 - window : 0);
    const int to0 = min(pos0, key_hi), to1 = min(pos1, key_hi);

    for (int kt = kt_begin; kt <= kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt < kt_end) load_kv(kt + 1, buf ^ 1);
        cp_async_commit();
        // the rows of the chunk after the next: its slot was last read by this chunk's copies, a barrier ago
        if (kt + 1 < kt_end) find_rows(kt + 2);
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kb = ks + buf * BN * KD;
        const __nv_bfloat16* vb = vs + buf * BN * DV;
        // a warp whose 16 rows lie past the block's rows (a single decoded token: all warps but one a map) only helps to load
        if (wrow >= rows) {
            __syncthreads();
            continue;
        }

        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            unsigned qf[4];
            ldmatrix_x4(qf, tile_ptr<KD>(qs, wrow + (lane & 15), mp * HD + kk * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int jp = 0; jp < BN / 16; ++jp) {
                unsigned b[4];
                const int mi = lane >> 3;
                ldmatrix_x4(b, tile_ptr<KD>((__nv_bfloat16*)kb, jp * 16 + (mi >> 1) * 8 + (lane & 7), mp * HD + kk * 16 + (mi & 1) * 8));
                mma_bf16(s[2 * jp], qf, b[0], b[1]);
                mma_bf16(s[2 * jp + 1], qf, b[2], b[3]);
            }
        }
        // the rows' ranges of keys and the running softmax
        const int kbase = kt * BN;
        unsigned ph[BN / 16][4], pl[BN / 16][4];
        {
            float mx0 = mrun[0], mx1 = mrun[1];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kbase + j * 8 + 2 * t4 + e;
                    const float a = (key >= from0 && key <= to0) ? s[j][e] * scale_log2 : -INFINITY;
                    const float b = (key >= from1 && key <= to1) ? s[j][2 + e] * scale_log2 : -INFINITY;
                    s[j][e] = a;
                    s[j][2 + e] = b;
                    mx0 = fmaxf(mx0, a);
                    mx1 = fmaxf(mx1, b);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float c0 = mx0 == -INFINITY ? 1.0f : exp2f(mrun[0] - mx0);
            const float c1 = mx1 == -INFINITY ? 1.0f : exp2f(mrun[1] - mx1);
            const float sub0 = mx0 == -INFINITY ? 0.0f : mx0, sub1 = mx1 == -INFINITY ? 0.0f : mx1;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                const float e0 = exp2f(s[j][0] - sub0), e1 = exp2f(s[j][1] - sub0);
                const float e2 = exp2f(s[j][2] - sub1), e3 = exp2f(s[j][3] - sub1);
                sum0 += e0 + e1;
                sum1 += e2 + e3;
                split_pair(e0, e1, ph[j >> 1][(j & 1) * 2], pl[j >> 1][(j & 1) * 2]);
                split_pair(e2, e3, ph[j >> 1][(j & 1) * 2 + 1], pl[j >> 1][(j & 1) * 2 + 1]);
            }
            lrun[0] = lrun[0] * c0 + sum0;
            lrun[1] = lrun[1] * c1 + sum1;
            mrun[0] = mx0;
            mrun[1] = mx1;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                o[i][0] *= c0; o[i][1] *= c0;
                o[i][2] *= c1; o[i][3] *= c1;
            }
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < DV / 16; ++dp) {
                unsigned b[4];
                const int mi = lane >> 3;
                ldmatrix_x4_trans(b, tile_ptr<DV>((__nv_bfloat16*)vb, kk * 16 + (mi & 1) * 8 + (lane & 7), dp * 16 + (mi >> 1) * 8));
                mma_bf16(o[2 * dp], ph[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], ph[kk], b[2], b[3]);
                mma_bf16(o[2 * dp], pl[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pl[kk], b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    float l0 = lrun[0], l1 = lrun[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int r0 = wrow + g, r1 = r0 + 8;
    if (partial) {
        // this stretch's share of both maps, unnormalised; the merge kernel finishes the rows
        const size_t per_row = (size_t)n_heads * 2 * (DV + 2);
        float* base = partial + ((size_t)blockIdx.z * T) * per_row + ((size_t)h * 2 + mp) * (DV + 2);
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            const int col = i * 8 + 2 * t4;
            if (r0 < rows) *(float2*)(base + (size_t)(row0 + r0) * per_row + col) = make_float2(o[i][0], o[i][1]);
            if (r1 < rows) *(float2*)(base + (size_t)(row0 + r1) * per_row + col) = make_float2(o[i][2], o[i][3]);
        }
        if (t4 == 0) {
            if (r0 < rows) *(float2*)(base + (size_t)(row0 + r0) * per_row + DV) = make_float2(mrun[0], l0);
            if (r1 < rows) *(float2*)(base + (size_t)(row0 + r1) * per_row + DV) = make_float2(mrun[1], l1);
        }
        return;
    }
    const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    // map 2's warps hand their rows over (the tiles of keys are done with: the loop ended on a barrier)
    float* a2 = (float*)ks;                                         // [BM][DV + 2] float32, over the tiles of keys and values
    static_assert((size_t)BM * (DV + 2) * sizeof(float) <= (size_t)2 * BN * (KD + DV) * sizeof(__nv_bfloat16), "room for map 2's rows");
    if (mp == 1) {
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            const int col = i * 8 + 2 * t4;
            *(float2*)(a2 + r0 * (DV + 2) + col) = make_float2(o[i][0] * i0, o[i][1] * i0);
            *(float2*)(a2 + r1 * (DV + 2) + col) = make_float2(o[i][2] * i1, o[i][3] * i1);
        }
    }
    __syncthreads();
    if (mp == 1) return;
    float ss0 = 0.0f, ss1 = 0.0f;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        const int col = i * 8 + 2 * t4;
        const float2 x0 = *(const float2*)(a2 + r0 * (DV + 2) + col), x1 = *(const float2*)(a2 + r1 * (DV + 2) + col);
        o[i][0] = o[i][0] * i0 - lambda * x0.x;
        o[i][1] = o[i][1] * i0 - lambda * x0.y;
        o[i][2] = o[i][2] * i1 - lambda * x1.x;
        o[i][3] = o[i][3] * i1 - lambda * x1.y;
        ss0 = fmaf(o[i][0], o[i][0], fmaf(o[i][1], o[i][1], ss0));
        ss1 = fmaf(o[i][2], o[i][2], fmaf(o[i][3], o[i][3], ss1));
    }
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
    const float n0 = out_scale / sqrtf(ss0 / (float)DV + eps), n1 = out_scale / sqrtf(ss1 / (float)DV + eps);
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        const int col = i * 8 + 2 * t4;
        if (r0 < rows) *(unsigned*)(out + ((size_t)(row0 + r0) * n_heads + h) * DV + col) = pack_bf16(o[i][0] * n0, o[i][1] * n0);
        if (r1 < rows) *(unsigned*)(out + ((size_t)(row0 + r1) * n_heads + h) * DV + col) = pack_bf16(o[i][2] * n1, o[i][3] * n1);
    }
}

// The stretches of a row's keys put together, map by map in stretch order, then the difference and the norm: a warp a
// (row, head).  Stretch z of a row at position p was written when z * split_keys <= p.
__global__ void __launch_bounds__(128) diff_merge_kernel(const float* __restrict__ partial, int splits, int split_keys, int T, int n_heads,
                                                         int vd, const int* __restrict__ positions, float lambda, float eps,
                                                         float out_scale, __nv_bfloat16* __restrict__ out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * 4 + warp;
    if (h >= n_heads) return;
    const int nz = min(splits, positions[t] / split_keys + 1);
    const size_t per_row = (size_t)n_heads * 2 * (vd + 2), per_split = (size_t)T * per_row;
    float a[2][4];                                   // vd <= 128: four entries a lane
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        const float* base = partial + (size_t)t * per_row + ((size_t)h * 2 + mp) * (vd + 2);
        float M = -INFINITY;
        for (int z = 0; z < nz; ++z) M = fmaxf(M, base[z * per_split + vd]);
        float L = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) a[mp][i] = 0.0f;
        for (int z = 0; z < nz; ++z) {
            const float mz = base[z * per_split + vd];
            const float f = mz == -INFINITY ? 0.0f : exp2f(mz - M);
            L = fmaf(f, base[z * per_split + vd + 1], L);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) a[mp][i] = fmaf(f, base[z * per_split + d], a[mp][i]);
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) a[mp][i] *= inv;
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a[0][i] = a[0][i] - lambda * a[1][i];
        ss = fmaf(a[0][i], a[0][i], ss);
    }
    ss = warp_sum(ss);
    const float norm = out_scale / sqrtf(ss / (float)vd + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) out[((size_t)t * n_heads + h) * vd + d] = __float2bfloat16_rn(a[0][i] * norm);
    }
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

// The tiled form: bfloat16 everywhere, hd in {32, 64, 128}, vd in {64, 128}.  tile_rows: 64, or 16 for steps in which no request
// brings more than 16 rows (single decoded tokens).  Request i owns rows [req_start[i], req_start[i+1])
// at positions req_prior[i] + j.  split_keys > 0 (a multiple of 64): a row block's keys are dealt to `splits` blocks in stretches
// of that many, partial [splits, T, n_heads, 2, vd + 2] float32 holds their shares, and a second kernel merges them.
CJ_EXPORT int cj_diff_attention_tile(const void* q, void* out, const void* kplane, const void* vplane, const int* positions,
                                     const int* req_start, const int* req_prior, int n_requests, int T, const int* table,
                                     int table_stride, int page_tokens, int n_heads, int n_kv, int hd, int vd, int window, float scale,
                                     float lambda, float eps, float out_scale, int split_keys, int splits, float* partial,
                                     int tile_rows, cudaStream_t stream) {
    if (T <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !req_start || !req_prior || !table) return CJ_ERR_ARG;
    if (n_heads <= 0 || n_heads > 65535 || n_kv <= 0 || n_heads % n_kv != 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (split_keys < 0 || split_keys % BN != 0 || (split_keys > 0 && (splits < 1 || splits > 65535 || !partial))) return CJ_ERR_ARG;
    if (tile_rows != 16 && tile_rows != 64) return CJ_ERR_SIZE;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid((T + tile_rows - 1) / tile_rows + n_requests, n_heads, split_keys > 0 ? splits : 1);
    float* part = split_keys > 0 ? partial : nullptr;
#define LAUNCH_M(H_, V_, M_)                                                                                             \
    {                                                                                                                    \
        size_t smem = (size_t)(M_ * 2 * H_ + 2 * BN * 2 * H_ + 2 * BN * V_) * sizeof(__nv_bfloat16);                     \
        static bool configured = false;                                                                                  \
        if (!configured) {                                                                                               \
            cudaError_t e = cudaFuncSetAttribute(diff_flash_kernel<H_, V_, M_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                         \
            configured = true;                                                                                           \
        }                                                                                                                \
        cj::launch_in_order(diff_flash_kernel<H_, V_, M_>, grid, dim3(M_ * 4), smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, \
                   (const __nv_bfloat16*)kplane, (const __nv_bfloat16*)vplane, req_start, req_prior, n_requests, T, table,  \
                   table_stride, page_tokens, n_heads, n_kv, window, scale_log2, lambda, eps, out_scale, split_keys, part); \
    }
#define LAUNCH(H_, V_)                                \
    {                                                 \
        if (tile_rows == 16) LAUNCH_M(H_, V_, 16)     \
        else LAUNCH_M(H_, V_, 64)                     \
    }
    if (hd == 32 && vd == 64) LAUNCH(32, 64)
    else if (hd == 32 && vd == 128) LAUNCH(32, 128)
    else if (hd == 64 && vd == 64) LAUNCH(64, 64)
    else if (hd == 64 && vd == 128) LAUNCH(64, 128)
    else if (hd == 128 && vd == 64) LAUNCH(128, 64)
    else if (hd == 128 && vd == 128) LAUNCH(128, 128)
    else return CJ_ERR_SIZE;
#undef LAUNCH_M
#undef LAUNCH
    if (split_keys > 0)
        cj::launch_in_order(diff_merge_kernel, dim3(T, (n_heads + 3) / 4), dim3(128), 0, stream, (const float*)part, splits, split_keys, T, n_heads,
                   vd, positions, lambda, eps, out_scale, (__nv_bfloat16*)out);
    return launch_status();
}
