// Attention over a compressed latent for steps that carry long prompt portions (bfloat16
// path): the plain form.  For the tokens of the step's requests the per-head keys
// k = [W_uk c | r] and values v = W_uv c are built once (two tensor-core products over the
// gathered latents) into dense buffers, and a query-tiled flash kernel runs over them:
// 64 query rows of one (request, head) against tiles of 64 keys, scores and weighted
// values on the tensor cores (mma.sync m16n8k16, bf16 in, f32 out), softmax statistics in
// float32 registers, keys and values through cp.async into swizzled shared memory, double
// buffered.  A (query, key, head) pair then costs 2 (dim + rot_dim + vdim) flops instead
// of the absorbed form's 2 (2 kv_rank + rot_dim), which pays as soon as a step has more
// than a few rows a request; decoding keeps the absorbed kernel, which reads a cache
// entry once for all heads.
//
//   latent_gather   c of every token of the step's requests (cached and new) -> [N, kv_rank]
//   latent_kv_pack  [N, H, DK] = [k_plain(h) | r | 0], [N, H, DV] = [v(h) | 0]   (DK, DV: padded to 64)
//   latent_q_pack   [T, H, DK] = [q_plain(h) | rotate(q_rot(h)) | 0]
//   latent_flash    out [T, H, DV]
//   latent_gate_rows out[t, h vdim + e] = o[t, h, e] * sigmoid(gate[t, h])
//
// Token n of the dense buffers is (request tok_req[n], position tok_pos[n]); request i's
// tokens lie at req_base[i] + position.  Rows are the step's rows: request i owns rows
// [req_start[i], req_start[i+1]) at positions req_prior[i] + j.
#define CJ_LIB "latent_prefill"
#include "common.cuh"

using namespace cj;

namespace {

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
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// element (row, col) of a [rows][D] bf16 tile whose 16-byte chunks are XOR-swizzled by row (D a multiple of 64)
template <int D>
__device__ __forceinline__ __nv_bfloat16* tile_ptr(__nv_bfloat16* base, int row, int col) {
    int chunk = (col >> 3) ^ (row & 7);
    return base + row * D + chunk * 8 + (col & 7);
}

constexpr int BM = 64, BN = 64, THREADS = 128;

template <int DK, int DV>
__global__ void __launch_bounds__(THREADS) latent_flash_kernel(
    const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ kx,
    const __nv_bfloat16* __restrict__ vx, const int* __restrict__ req_start, const int* __restrict__ req_prior,
    const int* __restrict__ req_base, int n_requests, int n_heads, float scale_log2, const float* __restrict__ sink) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* qs = (__nv_bfloat16*)smem_raw;                 // [BM][DK]
    __nv_bfloat16* ks = qs + BM * DK;                             // [2][BN][DK]
    __nv_bfloat16* vs = ks + 2 * BN * DK;                         // [2][BN][DV]
    constexpr int CK = DK / 8, CV = DV / 8;

    // which request and which tile of its rows; late tiles (the most keys) start first
    int tile = (int)gridDim.x - 1 - (int)blockIdx.x, req = -1, row0 = 0, rows = 0, first = 0;
    for (int r = 0; r < n_requests; ++r) {
        int lo = req_start[r], hi = req_start[r + 1];
        int tiles = (hi - lo + BM - 1) / BM;
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
    const int p0 = req_prior[req] + (row0 - req_start[req]);
    const int p_last = p0 + rows - 1;
    const int kt_end = p_last / BN;
    const long long base = req_base[req];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    auto load_kv = [&](int kt, int buf) {
        __nv_bfloat16* kd = ks + buf * BN * DK;
        __nv_bfloat16* vd = vs + buf * BN * DV;
        for (int i = tid; i < BN * CK; i += THREADS) {
            int r = i / CK, c = i % CK;
            int key = kt * BN + r;
            bool valid = key <= p_last;
            long long off = valid ? ((base + key) * n_heads + h) * DK + c * 8 : 0;
            cp_async16(kd + r * DK + (c ^ (r & 7)) * 8, kx + off, valid);
        }
        for (int i = tid; i < BN * CV; i += THREADS) {
            int r = i / CV, c = i % CV;
            int key = kt * BN + r;
            bool valid = key <= p_last;
            long long off = valid ? ((base + key) * n_heads + h) * DV + c * 8 : 0;
            cp_async16(vd + r * DV + (c ^ (r & 7)) * 8, vx + off, valid);
        }
    };
    for (int i = tid; i < BM * CK; i += THREADS) {
        int r = i / CK, c = i % CK;
        bool valid = r < rows;
        const __nv_bfloat16* src = q + ((size_t)(row0 + (valid ? r : 0)) * n_heads + h) * DK + c * 8;
        cp_async16(qs + r * DK + (c ^ (r & 7)) * 8, src, valid);
    }
    load_kv(0, 0);
    cp_async_commit();

    const int g = lane >> 2, t4 = lane & 3;
    const int wrow = warp * 16;
    float o[DV / 8][4];
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.0f, 0.0f};      // rows g and g + 8
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    for (int kt = 0; kt <= kt_end; ++kt) {
        const int buf = kt & 1;
        if (kt < kt_end) load_kv(kt + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* kb = ks + buf * BN * DK;
        const __nv_bfloat16* vb = vs + buf * BN * DV;

        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
            unsigned qf[4];
            ldmatrix_x4(qf, tile_ptr<DK>(qs, wrow + (lane & 15), kk * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int jp = 0; jp < BN / 16; ++jp) {
                unsigned b[4];
                int mi = lane >> 3;
                ldmatrix_x4(b, tile_ptr<DK>((__nv_bfloat16*)kb, jp * 16 + (mi >> 1) * 8 + (lane & 7), kk * 16 + (mi & 1) * 8));
                mma_bf16(s[2 * jp], qf, b[0], b[1]);
                mma_bf16(s[2 * jp + 1], qf, b[2], b[3]);
            }
        }
        // causal mask and running softmax
        const int kbase = kt * BN;
        unsigned pf[BN / 16][4];
        {
            const int pos0 = p0 + wrow + g, pos1 = pos0 + 8;
            float mx0 = mrun[0], mx1 = mrun[1];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    int key = kbase + j * 8 + 2 * t4 + e;
                    float a = key <= pos0 ? s[j][e] * scale_log2 : -INFINITY;
                    float b = key <= pos1 ? s[j][2 + e] * scale_log2 : -INFINITY;
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
                float e0 = exp2f(s[j][0] - sub0), e1 = exp2f(s[j][1] - sub0);
                float e2 = exp2f(s[j][2] - sub1), e3 = exp2f(s[j][3] - sub1);
                sum0 += e0 + e1;
                sum1 += e2 + e3;
                pf[j >> 1][(j & 1) * 2] = pack_bf16(e0, e1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(e2, e3);
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
                int mi = lane >> 3;
                ldmatrix_x4_trans(b, tile_ptr<DV>((__nv_bfloat16*)vb, kk * 16 + (mi & 1) * 8 + (lane & 7), dp * 16 + (mi >> 1) * 8));
                mma_bf16(o[2 * dp], pf[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pf[kk], b[2], b[3]);
            }
        }
        __syncthreads();
    }

    float l0 = lrun[0], l1 = lrun[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (sink) {
        // one more term of the divisor, without key or value: exp(sink), in the units of the running maximum (log 2)
        const float s2 = sink[h] * 1.4426950408889634f;
        l0 += exp2f(s2 - mrun[0]);
        l1 += exp2f(s2 - mrun[1]);
    }
    const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    const int r0 = wrow + g, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        int col = i * 8 + 2 * t4;
        if (r0 < rows) *(unsigned*)(out + ((size_t)(row0 + r0) * n_heads + h) * DV + col) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
        if (r1 < rows) *(unsigned*)(out + ((size_t)(row0 + r1) * n_heads + h) * DV + col) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
    }
}

__global__ void latent_gather_kernel(const __nv_bfloat16* __restrict__ plane, int width, int rank, const int* __restrict__ tok_req,
                                     const int* __restrict__ tok_pos, const int* __restrict__ table, int table_stride,
                                     int page_tokens, __nv_bfloat16* __restrict__ c_all) {
    cj::after_predecessor();
    cj::release_successor();
    const int n = blockIdx.x;
    const int pos = tok_pos[n];
    const int page = table[(size_t)tok_req[n] * table_stride + pos / page_tokens];
    const __nv_bfloat16* src = plane + ((size_t)page * page_tokens + pos % page_tokens) * width;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) c_all[(size_t)n * rank + e] = src[e];
}

__global__ void latent_kv_pack_kernel(const __nv_bfloat16* __restrict__ kp, const __nv_bfloat16* __restrict__ vp,
                                      const __nv_bfloat16* __restrict__ plane, int width, int rank, int rot,
                                      const int* __restrict__ tok_req, const int* __restrict__ tok_pos,
                                      const int* __restrict__ table, int table_stride, int page_tokens, int heads, int dim,
                                      int vdim, int DK, int DV, __nv_bfloat16* __restrict__ kx, __nv_bfloat16* __restrict__ vx) {
    cj::after_predecessor();
    cj::release_successor();
    const int n = blockIdx.x;
    const int pos = tok_pos[n];
    const int page = table[(size_t)tok_req[n] * table_stride + pos / page_tokens];
    const __nv_bfloat16* r = plane + ((size_t)page * page_tokens + pos % page_tokens) * width + rank;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
    for (int i = threadIdx.x; i < heads * DK; i += blockDim.x) {
        const int h = i / DK, e = i % DK;
        kx[(size_t)n * heads * DK + i] = e < dim ? kp[((size_t)n * heads + h) * dim + e] : (e < dim + rot ? r[e - dim] : zero);
    }
    for (int i = threadIdx.x; i < heads * DV; i += blockDim.x) {
        const int h = i / DV, e = i % DV;
        vx[(size_t)n * heads * DV + i] = e < vdim ? vp[((size_t)n * heads + h) * vdim + e] : zero;
    }
}

__global__ void latent_q_pack_kernel(const float* __restrict__ q, int ld, int heads, int dim, int rot, int rotary,
                                     const float* __restrict__ inv_freq, const int* __restrict__ positions, int DK,
                                     __nv_bfloat16* __restrict__ qx) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    const float* src = q + (size_t)r * ld;
    const int pos = positions[r];
    const int per = dim + rot;
    __nv_bfloat16* dst = qx + (size_t)r * heads * DK;
    for (int i = threadIdx.x; i < heads * DK; i += blockDim.x) {
        const int h = i / DK, e = i % DK;
        float v = 0.0f;
        if (e < dim) {
            v = src[h * per + e];
        } else if (e < dim + rotary) {
            const int j = e - dim, pair = j >> 1;
            const float a = (float)pos * inv_freq[pair];
            const float c = cosf(a), s = sinf(a);
            const float u = src[h * per + dim + 2 * pair], w = src[h * per + dim + 2 * pair + 1];
            v = (j & 1) ? w * c + u * s : u * c - w * s;
        } else if (e < per) {
            v = src[h * per + e];
        }
        dst[i] = __float2bfloat16_rn(v);
    }
}

__global__ void latent_gate_rows_kernel(const __nv_bfloat16* __restrict__ o, int DV, const float* __restrict__ gate, int ld_gate,
                                        int heads, int vdim, __nv_bfloat16* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
        const int h = i / vdim, e = i % vdim;
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)r * ld_gate + h])) : 1.0f;
        out[(size_t)r * heads * vdim + i] = __float2bfloat16_rn(__bfloat162float(o[((size_t)r * heads + h) * DV + e]) * g);
    }
}

}  // namespace

CJ_EXPORT int cj_latent_gather(const void* plane, int width, int rank, const int* tok_req, const int* tok_pos, const int* table,
                               int table_stride, int page_tokens, void* c_all, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (!plane || !tok_req || !tok_pos || !table || !c_all || rank <= 0 || width < rank || page_tokens <= 0) return CJ_ERR_ARG;
    cj::launch(latent_gather_kernel, dim3(N), dim3(rank >= 512 ? 256 : 128), 0, stream, (const __nv_bfloat16*)plane, width, rank,
               tok_req, tok_pos, table, table_stride, page_tokens, (__nv_bfloat16*)c_all);
    return launch_status();
}

CJ_EXPORT int cj_latent_kv_pack(const void* kp, const void* vp, const void* plane, int width, int rank, int rot, const int* tok_req,
                                const int* tok_pos, const int* table, int table_stride, int page_tokens, int heads, int dim,
                                int vdim, int DK, int DV, void* kx, void* vx, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (!kp || !vp || !plane || !tok_req || !tok_pos || !table || !kx || !vx) return CJ_ERR_ARG;
    if (DK < dim + rot || DV < vdim || width != rank + rot) return CJ_ERR_SIZE;
    cj::launch(latent_kv_pack_kernel, dim3(N), dim3(256), 0, stream, (const __nv_bfloat16*)kp, (const __nv_bfloat16*)vp,
               (const __nv_bfloat16*)plane, width, rank, rot, tok_req, tok_pos, table, table_stride, page_tokens, heads, dim, vdim,
               DK, DV, (__nv_bfloat16*)kx, (__nv_bfloat16*)vx);
    return launch_status();
}

CJ_EXPORT int cj_latent_q_pack(const float* q, int ld, int heads, int dim, int rot, int rotary, const float* inv_freq,
                               const int* positions, int DK, void* qx, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !positions || !qx || heads <= 0 || dim <= 0 || rot < 0 || DK < dim + rot) return CJ_ERR_ARG;
    if ((rotary & 1) || rotary < 0 || rotary > rot || (rotary > 0 && !inv_freq)) return CJ_ERR_SIZE;
    cj::launch(latent_q_pack_kernel, dim3(T), dim3(256), 0, stream, q, ld, heads, dim, rot, rotary, inv_freq, positions, DK,
               (__nv_bfloat16*)qx);
    return launch_status();
}

// q [T, heads, DK], kx [N, heads, DK], vx [N, heads, DV], out [T, heads, DV], all bf16; DK in {64, 128, 192, 256}, DV in {64, 128}
CJ_EXPORT int cj_latent_flash(const void* q, void* out, const void* kx, const void* vx, const int* req_start, const int* req_prior,
                              const int* req_base, int n_requests, int total_rows, int heads, int DK, int DV, float scale,
                              const float* sink, cudaStream_t stream) {
    if (total_rows <= 0 || n_requests <= 0) return 0;
    if (!q || !out || !kx || !vx || !req_start || !req_prior || !req_base) return CJ_ERR_ARG;
    if (heads <= 0 || heads > 65535) return CJ_ERR_SIZE;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid((total_rows + BM - 1) / BM + n_requests, heads);
#define LAUNCH(K_, V_)                                                                                                   \
    {                                                                                                                    \
        size_t smem = (size_t)(BM * K_ + 2 * BN * K_ + 2 * BN * V_) * sizeof(__nv_bfloat16);                             \
        static bool configured = false;                                                                                  \
        if (!configured) {                                                                                               \
            cudaError_t e = cudaFuncSetAttribute(latent_flash_kernel<K_, V_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                         \
            configured = true;                                                                                           \
        }                                                                                                                \
        cj::launch(latent_flash_kernel<K_, V_>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, \
                   (const __nv_bfloat16*)kx, (const __nv_bfloat16*)vx, req_start, req_prior, req_base, n_requests, heads, scale_log2, sink); \
        return launch_status();                                                                                          \
    }
    if (DV == 64) {
        if (DK == 64) LAUNCH(64, 64)
        if (DK == 128) LAUNCH(128, 64)
        if (DK == 192) LAUNCH(192, 64)
        if (DK == 256) LAUNCH(256, 64)
    } else if (DV == 128) {
        if (DK == 64) LAUNCH(64, 128)
        if (DK == 128) LAUNCH(128, 128)
        if (DK == 192) LAUNCH(192, 128)
        if (DK == 256) LAUNCH(256, 128)
    }
#undef LAUNCH
    return CJ_ERR_SIZE;
}

CJ_EXPORT int cj_latent_gate_rows(const void* o, int DV, const float* gate, int ld_gate, int heads, int vdim, void* out, int T,
                                  cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!o || !out || heads <= 0 || vdim <= 0 || DV < vdim) return CJ_ERR_ARG;
    cj::launch(latent_gate_rows_kernel, dim3(T), dim3(heads * vdim >= 2048 ? 256 : 128), 0, stream, (const __nv_bfloat16*)o, DV, gate,
               ld_gate, heads, vdim, (__nv_bfloat16*)out);
    return launch_status();
}
