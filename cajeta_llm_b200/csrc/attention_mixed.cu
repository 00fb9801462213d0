// Attention whose heads' scores are mixed before the softmax, with a sink, for bfloat16 storage: a tile of
// 16 query rows of one request and ALL heads, worked on by a thread-block cluster.
//
//   raw_g,ij = q_g,i . k_j                                         tensor cores (mma.sync, bf16 x bf16 -> f32)
//   s_h,ij   = sum_g talk[h, g] temp[g] scale raw_g,ij             float32, FMA units
//   o_h,i    = sum_j e^(s_h,ij - m) v_j / (sum_j e^(s_h,ij - m) + e^(sink_h - m))
// over the keys j of row i's window [p_i + 1 - w, p_i].  The mixing needs every head's raw score of a
// (row, key) pair, while the output accumulators of all heads (heads x 16 x vd float32) do not fit one SM.
// So the heads are dealt to the C blocks of a cluster, H / C <= 8 heads each, one head a warp: a block
// computes the raw scores of ITS heads for a chunk of 32 keys into its shared memory, the cluster meets,
// every block reads all blocks' raw scores through distributed shared memory and mixes them for its own
// output heads (a thread owns two adjacent keys of a row and all of the block's heads, so a raw score is
// read once per block and used for up to 8 products), and then each warp runs the running softmax and
// the weighted sum of values for its head.  A block loads only the key and value heads its own heads use.
// The softmax's weights stay float32 in effect: a weight enters the value product as two bfloat16 terms
// (its rounding and the rest), both accumulated in float32.  The sum over g runs in the order of g
// whatever C is, so the result does not depend on the cluster's size.  The cluster barrier is the
// hardware's (barrier.cluster): no block spins on memory.
//
// The sink is one more term e^(sink_h) of the divisor alone: sink_h is used as stored (scale and temp are for
// products of queries and keys), and nothing is added to the numerator.  So the running maximum starts at
// sink_h and the running sum at 1.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;
using namespace cj;

namespace {

constexpr int BM = 16;                // query rows a tile
constexpr int BN = 32;                // keys a chunk
constexpr int WARPS = 8;              // = the most heads a block owns
constexpr int THREADS = WARPS * 32;
constexpr int KT_MAX = 8;             // 16-wide steps over a head's size: hd <= 128
constexpr int VT_MAX = 16;            // 8-wide tiles over a value's size: vd <= 128
constexpr int RS = BN + 8;            // row stride of a score tile, floats
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// a pair of float32 as (rounded to bf16, the rest rounded to bf16), each pair packed in a word
__device__ __forceinline__ void split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);              // one conversion for the pair
    hi = *(const uint32_t*)&h;
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - __uint_as_float(hi << 16), y - __uint_as_float(hi & 0xffff0000u));
    lo = *(const uint32_t*)&l;
}
// 2^x by the special-function unit alone (relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// the key/value heads that the heads [g_lo, g_lo + hl) use
__host__ __device__ inline void kv_range(int g_lo, int hl, int per_kv, int& kv_lo, int& n) {
    kv_lo = g_lo / per_kv;
    n = (g_lo + hl - 1) / per_kv - kv_lo + 1;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16 bytes global -> shared without a register in between; not valid: the 16 bytes become zeros
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// four 8x8 bf16 matrices, lane l gives the address of row l % 8 of matrix l / 8
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}

// FULL: heads and values of 128 and 8 heads a block, known to the compiler: the generic loops' guards fall away.
template <bool FULL>
__global__ void __launch_bounds__(THREADS, 2) mixed_heads_tile_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ kplane, const bf16* __restrict__ vplane,
    const int* __restrict__ positions, const int* __restrict__ req_start, int n_requests, const int* __restrict__ table,
    int table_stride, int page_tokens, int n_heads, int n_kv, int hd_given, int vd_given, int window, float scale,
    const float* __restrict__ temp, const float* __restrict__ talk, const float* __restrict__ sink, int kv_local_max,
    float* __restrict__ partial, int total_rows) {
    cj::after_predecessor();
    cj::release_successor();
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    const int hd = FULL ? 128 : hd_given, vd = FULL ? 128 : vd_given;
    const int HL = FULL ? WARPS : n_heads / C, g_lo = crank * HL, per_kv = n_heads / n_kv;
    int kv_lo, nkvl;
    kv_range(g_lo, HL, per_kv, kv_lo, nkvl);
    const int hdp = (hd + 15) & ~15, KT = hdp / 16, VT = vd / 8, KS = hdp + 8, VR = vd + 8;

    // ---- which request and which 16-row tile of it: the same for every block of the cluster ----
    int tile = (int)(gridDim.x / C) - 1 - (int)(blockIdx.x / C), req = -1, row0 = 0, rows = 0, first = 0;
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

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* raw = (float*)smem_raw;                         // [HL][BM][RS] raw scores of this block's heads
    float* mixed = raw + HL * BM * RS;                     // [HL][BM][RS] mixed scores of this block's heads
    float* ct = mixed + HL * BM * RS;                      // [n_heads][8]: what raw head g gives to local head u
    bf16* qs = (bf16*)(ct + n_heads * 8);                  // [HL][BM][KS]
    bf16* ks = qs + (size_t)HL * BM * KS;                  // [kv_local_max][BN][KS]
    bf16* vs = ks + (size_t)kv_local_max * BN * KS;        // [kv_local_max][BN][VR]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
    const int p0 = positions[row0], p_last = p0 + rows - 1;
    const int key_from = (window > 0 && p0 + 1 > window) ? p0 + 1 - window : 0;
    const int n_chunks = (p_last - key_from) / BN + 1;
    // the keys may be dealt to gridDim.y clusters, a stretch of chunks each: then every one leaves (o, m, l) for the merge
    const int splits = (int)gridDim.y, split = (int)blockIdx.y;
    const int per_split = (n_chunks + splits - 1) / splits;
    const int c_begin = min(n_chunks, split * per_split), c_end = min(n_chunks, c_begin + per_split);
    const int* tab = table + (size_t)req * table_stride;

    for (int i = tid; i < n_heads * 8; i += THREADS) {
        const int g = i >> 3, u = i & 7;
        float c = 0.0f;
        if (u < HL) {
            c = talk ? talk[(size_t)(g_lo + u) * n_heads + g] : (g == g_lo + u ? 1.0f : 0.0f);
            c *= scale * (temp ? temp[g] : 1.0f) * LOG2E;      // mixed scores come out in units of log 2: e^s = 2^(s log2 e)
        }
        ct[i] = c;
    }
    {   // the stretch of a query or key row past hd enters the products: zeros, not whatever lay there
        uint32_t* z = (uint32_t*)qs;
        const int words = (HL * BM + kv_local_max * BN) * KS / 2;
        for (int i = tid; i < words; i += THREADS) z[i] = 0u;
    }
    __syncthreads();

    const int ch_k = hd / 8;
    __shared__ long long place[2][BN];                     // a chunk's keys in the planes, in (token, kv head 0) entries; -1: none
    auto find_places = [&](int c) {                        // by the first warp; read after the block's next meeting
        if (tid < BN) {
            const int key = key_from + c * BN + tid;
            long long at = -1;
            if (c < c_end && key <= p_last) {
                const int page = tab[key / page_tokens];
                if (page >= 0) at = (long long)page * n_kv * page_tokens + key % page_tokens;
            }
            place[c & 1][tid] = at;
        }
    };
    auto load_keys = [&](int c) {
        const long long* at = place[c & 1];
        for (int kv = 0; kv < nkvl; ++kv)
            for (int i = tid; i < BN * ch_k; i += THREADS) {
                const int r = i / ch_k, ch = i - r * ch_k;
                const bool valid = at[r] >= 0;
                cp_async16(ks + ((size_t)kv * BN + r) * KS + ch * 8,
                           kplane + (valid ? ((size_t)at[r] + (size_t)(kv_lo + kv) * page_tokens) * hd + ch * 8 : 0), valid);
            }
    };
    auto load_values = [&](int c) {
        const long long* at = place[c & 1];
        for (int kv = 0; kv < nkvl; ++kv)
            for (int i = tid; i < BN * VT; i += THREADS) {
                const int r = i / VT, ch = i - r * VT;
                const bool valid = at[r] >= 0;
                cp_async16(vs + ((size_t)kv * BN + r) * VR + ch * 8,
                           vplane + (valid ? ((size_t)at[r] + (size_t)(kv_lo + kv) * page_tokens) * vd + ch * 8 : 0), valid);
            }
    };
    find_places(c_begin);
    __syncthreads();
    // the tile's queries of this block's heads, then the first chunk's keys, then its values: three groups
    for (int i = tid; i < HL * BM * ch_k; i += THREADS) {
        const int ch = i % ch_k, r = (i / ch_k) % BM, u = i / (ch_k * BM);
        const bool valid = r < rows;
        cp_async16(qs + ((size_t)u * BM + r) * KS + ch * 8, q + ((size_t)(row0 + (valid ? r : 0)) * n_heads + g_lo + u) * hd + ch * 8, valid);
    }
    cp_async_commit();
    load_keys(c_begin);
    cp_async_commit();
    load_values(c_begin);
    cp_async_commit();

    // ---- this warp's head: running maximum and sum, output accumulators ----
    const bool has_head = warp < HL;
    const int head = g_lo + warp;
    float o[VT_MAX][4];
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
#pragma unroll
    for (int v = 0; v < VT_MAX; ++v) o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.0f;
    if (has_head && sink && split == 0) {
        m0 = m1 = sink[head] * LOG2E;
        l0 = l1 = 1.0f;
    }
    const int kvl = has_head ? head / per_kv - kv_lo : 0;
    // ldmatrix addresses: a lane's row and column within a 16 x 16 stretch
    const bf16* q_lane = qs + ((size_t)warp * BM + (lane & 7) + ((lane >> 3) & 1) * 8) * KS + (lane >> 4) * 8;
    const bf16* k_lane = ks + ((size_t)kvl * BN + (lane & 7) + (lane >> 4) * 8) * KS + ((lane >> 3) & 1) * 8;
    const bf16* v_lane = vs + ((size_t)kvl * BN + (lane & 7) + ((lane >> 3) & 1) * 8) * VR + (lane >> 4) * 8;

    for (int c = c_begin; c < c_end; ++c) {
        const int key0 = key_from + c * BN;
        find_places(c + 1);                                // read from the cluster's meeting below on
        cp_async_wait<1>();                                // the chunk's keys (and the queries) have arrived; its values may be on the way
        __syncthreads();
        if (c > c_begin) cluster_wait();                         // every block has read the last chunk's raw scores

        // ---- raw scores of this warp's head ----
        if (has_head) {
            float acc[BN / 8][4];
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
#pragma unroll
            for (int kt = 0; kt < KT_MAX; ++kt) {
                if (kt < KT) {
                    uint32_t a[4], b[4];
                    ldsm_x4(a, q_lane + kt * 16);
#pragma unroll
                    for (int np = 0; np < BN / 16; ++np) {
                        ldsm_x4(b, k_lane + (size_t)np * 16 * KS + kt * 16);
                        mma_bf16(acc[2 * np], a, b[0], b[1]);
                        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
                *(float2*)(raw + ((size_t)warp * BM + r0) * RS + nt * 8 + cq) = make_float2(acc[nt][0], acc[nt][1]);
                *(float2*)(raw + ((size_t)warp * BM + r1) * RS + nt * 8 + cq) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
        cluster_arrive();
        cluster_wait();                                    // all heads' raw scores of the chunk are written; the keys are free
        load_keys(c + 1);                                  // the next chunk's keys travel while this one is mixed and summed
        cp_async_commit();

        // ---- mixing: a thread owns two adjacent keys of a row, and the block's heads ----
        {
            const int i = tid >> 4, j = (tid & 15) * 2;
            float2 a[8];                                   // packed: one instruction multiplies a coefficient into both keys
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = make_float2(0.0f, 0.0f);
            for (int rr = 0; rr < C; ++rr) {
                const float* theirs = cluster.map_shared_rank(raw, rr) + (size_t)i * RS + j;
                float2 x[8];
#pragma unroll
                for (int gl = 0; gl < 8; ++gl) x[gl] = gl < HL ? *(const float2*)(theirs + (size_t)gl * BM * RS) : make_float2(0.0f, 0.0f);
#pragma unroll
                for (int gl = 0; gl < 8; ++gl) {
                    if (gl < HL) {
                        const float4 c0 = *(const float4*)(ct + (size_t)(rr * HL + gl) * 8);
                        const float4 c1 = *(const float4*)(ct + (size_t)(rr * HL + gl) * 8 + 4);
                        a[0] = __ffma2_rn(make_float2(c0.x, c0.x), x[gl], a[0]);
                        a[1] = __ffma2_rn(make_float2(c0.y, c0.y), x[gl], a[1]);
                        a[2] = __ffma2_rn(make_float2(c0.z, c0.z), x[gl], a[2]);
                        a[3] = __ffma2_rn(make_float2(c0.w, c0.w), x[gl], a[3]);
                        a[4] = __ffma2_rn(make_float2(c1.x, c1.x), x[gl], a[4]);
                        a[5] = __ffma2_rn(make_float2(c1.y, c1.y), x[gl], a[5]);
                        a[6] = __ffma2_rn(make_float2(c1.z, c1.z), x[gl], a[6]);
                        a[7] = __ffma2_rn(make_float2(c1.w, c1.w), x[gl], a[7]);
                    }
                }
            }
            const int p_i = p0 + min(i, rows - 1);
            const int ka = key0 + j, kb = ka + 1;
            const bool va = ka <= p_i && (window <= 0 || ka > p_i - window);
            const bool vb = kb <= p_i && (window <= 0 || kb > p_i - window);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (u < HL)
                    *(float2*)(mixed + ((size_t)u * BM + i) * RS + j) = make_float2(va ? a[u].x : -INFINITY, vb ? a[u].y : -INFINITY);
            // done with the other blocks' raw scores: what was read has been used, and nothing this block wrote since
            // the last meeting is for another block to see, so the arrival orders no memory
            cluster_arrive_relaxed();
        }
        cp_async_wait<1>();                                // the chunk's values have arrived; the next keys may be on the way
        __syncthreads();

        // ---- running softmax and the weighted sum of values of this warp's head ----
        if (has_head) {
            float2 s0[BN / 8], s1[BN / 8];
            float x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
            for (int t = 0; t < BN / 8; ++t) {
                s0[t] = *(const float2*)(mixed + ((size_t)warp * BM + r0) * RS + t * 8 + cq);
                s1[t] = *(const float2*)(mixed + ((size_t)warp * BM + r1) * RS + t * 8 + cq);
                x0 = fmaxf(x0, fmaxf(s0[t].x, s0[t].y));
                x1 = fmaxf(x1, fmaxf(s1[t].x, s1[t].y));
            }
            const float n0 = fmaxf(m0, quad_max(x0)), n1 = fmaxf(m1, quad_max(x1));
            const float u0 = n0 == -INFINITY ? 0.0f : n0, u1 = n1 == -INFINITY ? 0.0f : n1;   // nothing seen yet: all terms 0
            const float f0 = ex2(m0 - u0), f1 = ex2(m1 - u1);
            float e0 = 0.0f, e1 = 0.0f;
#pragma unroll
            for (int t = 0; t < BN / 8; ++t) {
                s0[t].x = ex2(s0[t].x - u0); s0[t].y = ex2(s0[t].y - u0);
                s1[t].x = ex2(s1[t].x - u1); s1[t].y = ex2(s1[t].y - u1);
                e0 += s0[t].x + s0[t].y;
                e1 += s1[t].x + s1[t].y;
            }
            l0 = l0 * f0 + quad_sum(e0);
            l1 = l1 * f1 + quad_sum(e1);
            m0 = n0;
            m1 = n1;
            if (f0 != 1.0f || f1 != 1.0f) {
#pragma unroll
                for (int v = 0; v < VT_MAX; ++v) { o[v][0] *= f0; o[v][1] *= f0; o[v][2] *= f1; o[v][3] *= f1; }
            }
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t hi[4], lo[4], b[4];
                split_pair(s0[2 * kk].x, s0[2 * kk].y, hi[0], lo[0]);
                split_pair(s1[2 * kk].x, s1[2 * kk].y, hi[1], lo[1]);
                split_pair(s0[2 * kk + 1].x, s0[2 * kk + 1].y, hi[2], lo[2]);
                split_pair(s1[2 * kk + 1].x, s1[2 * kk + 1].y, hi[3], lo[3]);
                // four tiles of the value's size at a time, the rounded weights first and the rest after: two products into
                // one accumulator are four instructions apart
#pragma unroll
                for (int v = 0; v < VT_MAX; v += 4) {
                    if (v < VT) {
                        uint32_t b2[4];
                        ldsm_x4_trans(b, v_lane + (size_t)kk * 16 * VR + v * 8);
                        if (v + 2 < VT) ldsm_x4_trans(b2, v_lane + (size_t)kk * 16 * VR + (v + 2) * 8);
                        mma_bf16(o[v], hi, b[0], b[1]);
                        if (v + 1 < VT) mma_bf16(o[v + 1], hi, b[2], b[3]);
                        if (v + 2 < VT) mma_bf16(o[v + 2], hi, b2[0], b2[1]);
                        if (v + 3 < VT) mma_bf16(o[v + 3], hi, b2[2], b2[3]);
                        mma_bf16(o[v], lo, b[0], b[1]);
                        if (v + 1 < VT) mma_bf16(o[v + 1], lo, b[2], b[3]);
                        if (v + 2 < VT) mma_bf16(o[v + 2], lo, b2[0], b2[1]);
                        if (v + 3 < VT) mma_bf16(o[v + 3], lo, b2[2], b2[3]);
                    }
                }
            }
        }
        __syncthreads();                                   // the chunk's values and mixed scores are free again
        load_values(c + 1);
        cp_async_commit();
    }
    cp_async_wait<0>();
    if (c_end > c_begin) cluster_wait();                   // no block leaves while another may still read its raw scores

    if (partial) {
        // [split][row][head][vd + 2]: the sum of weighted values as it stands, then the maximum (in units of log 2) and the sum
        if (has_head) {
            float* d0 = partial + (((size_t)split * total_rows + row0 + r0) * n_heads + head) * (vd + 2);
            float* d1 = partial + (((size_t)split * total_rows + row0 + r1) * n_heads + head) * (vd + 2);
#pragma unroll
            for (int v = 0; v < VT_MAX; ++v) {
                if (v < VT) {
                    if (r0 < rows) *(float2*)(d0 + v * 8 + cq) = make_float2(o[v][0], o[v][1]);
                    if (r1 < rows) *(float2*)(d1 + v * 8 + cq) = make_float2(o[v][2], o[v][3]);
                }
            }
            if ((lane & 3) == 0) {
                if (r0 < rows) { d0[vd] = m0; d0[vd + 1] = l0; }
                if (r1 < rows) { d1[vd] = m1; d1[vd + 1] = l1; }
            }
        }
        return;
    }

    if (has_head) {
        const float i0 = 1.0f / l0, i1 = 1.0f / l1;
        bf16* o0 = out + ((size_t)(row0 + r0) * n_heads + head) * vd + cq;
        bf16* o1 = out + ((size_t)(row0 + r1) * n_heads + head) * vd + cq;
#pragma unroll
        for (int v = 0; v < VT_MAX; ++v) {
            if (v < VT) {
                if (r0 < rows) *(__nv_bfloat162*)(o0 + v * 8) = __floats2bfloat162_rn(o[v][0] * i0, o[v][1] * i0);
                if (r1 < rows) *(__nv_bfloat162*)(o1 + v * 8) = __floats2bfloat162_rn(o[v][2] * i1, o[v][3] * i1);
            }
        }
    }
}

// One warp a (row, head): the clusters' shares of the keys are put together, o = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s.
__global__ void __launch_bounds__(128) mixed_heads_merge_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int splits,
                                                                int total_rows, int n_heads, int vd) {
    cj::after_predecessor();
    cj::release_successor();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);                 // row * n_heads + head
    if (item >= total_rows * n_heads) return;
    const size_t each = (size_t)total_rows * n_heads * (vd + 2);
    const float* p = partial + (size_t)item * (vd + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * each + vd]);
    float L = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float m = p[s * each + vd];
        if (m != -INFINITY) L = fmaf(p[s * each + vd + 1], exp2f(m - M), L);
    }
    for (int d = lane; d < vd; d += 32) {
        float a = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float m = p[s * each + vd];
            if (m != -INFINITY) a = fmaf(p[s * each + d], exp2f(m - M), a);
        }
        out[(size_t)item * vd + d] = __float2bfloat16_rn(a / L);
    }
}

// the cluster's size for these heads: the smallest of 1, 2, 4, 8 that leaves a block at most 8 heads; 0: none
inline int cluster_for(int n_heads) {
    for (int c = 1; c <= 8; c *= 2)
        if (n_heads % c == 0 && n_heads / c <= WARPS) return c;
    return 0;
}

inline size_t tile_smem(int n_heads, int n_kv, int hd, int vd, int C, int& kv_local_max) {
    const int HL = n_heads / C, per_kv = n_heads / n_kv, hdp = (hd + 15) & ~15;
    kv_local_max = 1;
    for (int r = 0; r < C; ++r) {
        int lo, n;
        kv_range(r * HL, HL, per_kv, lo, n);
        if (n > kv_local_max) kv_local_max = n;
    }
    return (size_t)2 * HL * BM * RS * sizeof(float) + (size_t)n_heads * 8 * sizeof(float) + (size_t)HL * BM * (hdp + 8) * sizeof(bf16) +
           (size_t)kv_local_max * BN * (hdp + 8) * sizeof(bf16) + (size_t)kv_local_max * BN * (vd + 8) * sizeof(bf16);
}

}  // namespace

// 1 if the tiled form takes these sizes (bfloat16 storage, head and value sizes multiples of 8 up to 128,
// heads that a cluster of at most 8 blocks can deal out 8 a block), else 0: the caller then uses the
// row-at-a-time form.
CJ_EXPORT int cj_mixed_heads_tile_fits(int n_heads, int n_kv, int hd, int vd) {
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0) return 0;
    if (hd <= 0 || vd <= 0 || hd % 8 != 0 || vd % 8 != 0 || hd > 16 * KT_MAX || vd > 8 * VT_MAX) return 0;
    const int C = cluster_for(n_heads);
    if (C == 0) return 0;
    int kvm;
    return tile_smem(n_heads, n_kv, hd, vd, C, kvm) <= 200 * 1024 ? 1 : 0;
}

// q [T, n_heads, hd], out [T, n_heads, vd], planes [pages, n_kv, page_tokens, hd | vd]: bfloat16.  req_start
// [n_requests + 1]: the rows of request r are [req_start[r], req_start[r + 1]), at consecutive positions.
// temp [n_heads], talk [n_heads, n_heads], sink [n_heads]: float32 or null.  cluster_blocks: 0 = chosen here, else the cluster's
// size (a power of two up to 8 that divides n_heads and leaves a block at most 8 heads).  splits > 1: a tile's chunks of keys are
// dealt to that many clusters, which leave their shares in partial, float32 [splits, total_rows, n_heads, vd + 2], and a second
// kernel puts them together: for steps of few rows (single decoded tokens), where a tile's chunks would run one after the other.
CJ_EXPORT int cj_mixed_heads_attention_tile(const void* q, void* out, const void* kplane, const void* vplane, const int* positions,
                                            const int* req_start, int n_requests, int total_rows, const int* table, int table_stride,
                                            int page_tokens, int n_heads, int n_kv, int hd, int vd, int window, float scale,
                                            const float* temp, const float* talk, const float* sink, int cluster_blocks, float* partial, int splits,
                                            cudaStream_t stream) {
    if (total_rows <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kplane || !vplane || !positions || !req_start || !table) return CJ_ERR_ARG;
    if (!cj_mixed_heads_tile_fits(n_heads, n_kv, hd, vd) || page_tokens <= 0) return CJ_ERR_SIZE;
    const int tiles = (total_rows + BM - 1) / BM + n_requests;
    int C = cluster_for(n_heads);
    if (cluster_blocks > 0) {
        if ((cluster_blocks & (cluster_blocks - 1)) || cluster_blocks > 8 || n_heads % cluster_blocks || n_heads / cluster_blocks > WARPS) return CJ_ERR_SIZE;
        C = cluster_blocks;
    }
    int kvm;
    const size_t smem = tile_smem(n_heads, n_kv, hd, vd, C, kvm);
    static size_t sized = 48 * 1024;
    if (smem > sized) {
        cudaError_t e = cudaFuncSetAttribute(mixed_heads_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(mixed_heads_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        sized = smem;
    }
    cudaLaunchConfig_t cfg = {};
    if (splits < 1 || (splits > 1 && !partial)) return CJ_ERR_ARG;
    cfg.gridDim = dim3(tiles * C, splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool full = hd == 128 && vd == 128 && n_heads / C == WARPS;
    cudaLaunchKernelEx(&cfg, full ? mixed_heads_tile_kernel<true> : mixed_heads_tile_kernel<false>, (const bf16*)q, (bf16*)out,
                       (const bf16*)kplane, (const bf16*)vplane, positions, req_start, n_requests, table, table_stride, page_tokens,
                       n_heads, n_kv, hd, vd, window, scale, temp, talk, sink, kvm, splits > 1 ? partial : (float*)nullptr, total_rows);
    if (splits > 1)
        cj::launch(mixed_heads_merge_kernel, dim3((total_rows * n_heads + 3) / 4), dim3(128), 0, stream, (const float*)partial, (bf16*)out,
                   splits, total_rows, n_heads, vd);
    return launch_status();
}
