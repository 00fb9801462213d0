// Attention over a compressed latent.  A token's cache entry is one vector shared by all
// heads: the normed latent c (kv_rank entries) followed by one rotated key part (rot_dim
// entries).  Head h's unrotated key is W_uk[h] c and its value W_uv[h] c; both products are
// moved to the query's side, so that nothing per head is ever built from the cache:
//
//   score[h, j] = ((W_uk[h]^T q_plain[h]) . c_j + q_rot[h] . r_j) * scale
//   out[h]      = W_uv[h] (sum_j softmax(score[h])_j c_j)
//
// latent_kv_write   c = rms(d[:kv_rank]) * w, r = rotate(d[kv_rank:]) -> the row's place in the paged cache
// latent_q_split    q [T, H (dim + rot_dim)] -> q_plain [H, T, dim] (head-major, the grouped product's
//                   input) and the rotated parts [T, H, rot_dim] in float32
// latent_attention  scores, softmax and the weighted sum of latents for every (row, head);
//                   q_abs [H, T, kv_rank] in, the summed latents [H, T, kv_rank] out (both head-major;
//                   the sums leave in the cache's dtype, as the next product's input)
// latent_gate_out   out[t, h, :] = o[h, t, :] * sigmoid(gate[t, h])  (back to token-major; without a gate: the move alone)
// latent_q_norm     the queries' own latent: rms(x[:, offset : offset + n]) * w into the activation dtype
//
// A sink (optional, one float32 per head): the softmax's divisor also holds exp(sink[h]), a term without key or value
// that is neither scaled nor rotated; the running maximum of a row's first stretch starts at it and the running sum at 1.
//
// The rotation pairs entries (2i, 2i+1); the angle p * inv_freq[i] is float32.  Scores,
// softmax and sums are float32 whatever the cache holds.
#define CJ_LIB "latent_attention"
#include "common.cuh"

using namespace cj;

namespace {

template <typename TC>
__global__ void latent_kv_write_kernel(const float* __restrict__ d, int ld, int rank, int rot, int rotary, const float* __restrict__ w,
                                       float eps, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                       const int* __restrict__ row_req, const int* __restrict__ table, int table_stride,
                                       int page_tokens, TC* __restrict__ plane) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* src = d + (size_t)r * ld;
    const int pos = positions[r];
    const int page = table[(size_t)row_req[r] * table_stride + pos / page_tokens];
    TC* dst = plane + ((size_t)page * page_tokens + pos % page_tokens) * (rank + rot);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < nw; ++i) total += scratch[i];
    const float scale = 1.0f / sqrtf(total / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<TC>(src[i] * scale * w[i]);
    for (int i = threadIdx.x; i < rotary / 2; i += blockDim.x) {
        const float a = (float)pos * inv_freq[i];
        const float c = cosf(a), s = sinf(a);
        const float u = src[rank + 2 * i], v = src[rank + 2 * i + 1];
        dst[rank + 2 * i] = from_f32<TC>(u * c - v * s);
        dst[rank + 2 * i + 1] = from_f32<TC>(v * c + u * s);
    }
    for (int i = rotary + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = from_f32<TC>(src[rank + i]);   // past the rotated dims: unchanged
}

template <typename TO>
__global__ void latent_q_split_kernel(const float* __restrict__ q, int ld, int heads, int dim, int rot, int rotary,
                                      const float* __restrict__ inv_freq, const int* __restrict__ positions, int T,
                                      TO* __restrict__ q_plain, float* __restrict__ q_rot) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    const float* src = q + (size_t)r * ld;
    const int pos = positions[r];
    const int per = dim + rot;
    for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
        const int h = i / dim, e = i % dim;
        q_plain[((size_t)h * T + r) * dim + e] = from_f32<TO>(src[h * per + e]);
    }
    for (int i = threadIdx.x; i < heads * (rotary / 2); i += blockDim.x) {
        const int h = i / (rotary / 2), e = i % (rotary / 2);
        const float a = (float)pos * inv_freq[e];
        const float c = cosf(a), s = sinf(a);
        const float u = src[h * per + dim + 2 * e], v = src[h * per + dim + 2 * e + 1];
        float* dst = q_rot + ((size_t)r * heads + h) * rot;
        dst[2 * e] = u * c - v * s;
        dst[2 * e + 1] = v * c + u * s;
    }
    const int rest = rot - rotary;
    for (int i = threadIdx.x; i < heads * rest; i += blockDim.x) {
        const int h = i / rest, e = rotary + i % rest;
        q_rot[((size_t)r * heads + h) * rot + e] = src[h * per + dim + e];
    }
}

// One block: one row, up to 8 heads (a warp each), one stretch of the row's keys.  Keys come
// in chunks of 32 into shared memory (a row of the chunk is padded to an odd number of 32-bit
// words, so that 32 lanes reading 32 keys at one offset hit 32 banks); lane j of a warp scores
// key j for the warp's head, the warp keeps the running maximum and sum, and for the weighted
// sum a lane owns entries of the latent at a stride of 32 (pairs of them at a stride of 64
// when the cache holds 16-bit entries: one 32-bit word a read).
// With few rows in the step (decoding) the keys of a row are cut into stretches of split_keys,
// one block each (blockIdx.z), which leave unnormalised sums, maxima and weights behind; a
// second kernel merges them in stretch order.  How a row is cut depends on its position and
// split_keys only.
constexpr int LA_KEYS = 32;
constexpr int LA_HEADS = 8;

template <typename TC> struct Packed { static constexpr bool value = false; };
template <> struct Packed<__nv_bfloat16> { static constexpr bool value = true; };

template <typename TC, int NACC>
__global__ void __launch_bounds__(LA_HEADS * 32) latent_attention_kernel(
    const float* __restrict__ q_abs, const float* __restrict__ q_rot, const TC* __restrict__ plane, int rank, int rot,
    int heads, int T, const int* __restrict__ positions, const int* __restrict__ row_req, const int* __restrict__ table,
    int table_stride, int page_tokens, float scale, TC* __restrict__ out, int row_words, int split_keys,
    float* __restrict__ part_acc, float* __restrict__ part_ml, const float* __restrict__ sink) {
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(16) unsigned char smem[];
    const int width = rank + rot;
    float* qs = (float*)smem;                                   // [LA_HEADS][width]
    float* ps = qs + LA_HEADS * width;                          // [LA_HEADS][LA_KEYS]
    uint32_t* ks = (uint32_t*)(ps + LA_HEADS * LA_KEYS);        // [LA_KEYS][row_words]
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * LA_HEADS + warp;
    const bool has_head = head < heads;
    const int pos = positions[r];
    const int key_begin = split_keys > 0 ? (int)blockIdx.z * split_keys : 0;
    const int key_end = split_keys > 0 ? min(pos + 1, key_begin + split_keys) : pos + 1;
    if (key_begin >= key_end) return;                            // this stretch lies past the row's position
    const int* pages = table + (size_t)row_req[r] * table_stride;
    if (has_head) {
        const float* qa = q_abs + ((size_t)head * T + r) * rank;
        const float* qr = q_rot + ((size_t)r * heads + head) * rot;
        for (int i = lane; i < rank; i += 32) qs[warp * width + i] = qa[i];
        for (int i = lane; i < rot; i += 32) qs[warp * width + rank + i] = qr[i];
    }
    // 16-bit entries, an even number of them in the latent and in the whole entry: two a word
    const bool packed = Packed<TC>::value && (rank % 2 == 0) && (width % 2 == 0);
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    if (sink && has_head && key_begin == 0) { m = sink[head]; l = 1.0f; }       // the sink counts once: in the row's first stretch
    const TC* krow_base = (const TC*)ks;
    const int row_elems = row_words * (int)(4 / sizeof(TC));
    for (int k0 = key_begin; k0 < key_end; k0 += LA_KEYS) {
        const int n_keys = min(LA_KEYS, key_end - k0);
        __syncthreads();                                        // the chunk before has been used up (and qs is written)
        // bring the chunk in: a key's entry is contiguous in its page.  A warp brings four keys
        // (warp, warp + 8, ...), their loads side by side: four independent round trips in flight
        // a pass instead of one.
        {
            constexpr int PER_WARP = LA_KEYS / LA_HEADS;
            const TC* srcs[PER_WARP];
#pragma unroll
            for (int u = 0; u < PER_WARP; ++u) {
                const int j = warp + LA_HEADS * u;
                const int kp = k0 + (j < n_keys ? j : 0);
                srcs[u] = plane + ((size_t)pages[kp / page_tokens] * page_tokens + kp % page_tokens) * width;
            }
            if ((width * sizeof(TC)) % 4 == 0) {
                const int words = width * (int)sizeof(TC) / 4;
                for (int e = lane; e < words; e += 32) {
                    uint32_t v[PER_WARP];
#pragma unroll
                    for (int u = 0; u < PER_WARP; ++u) v[u] = warp + LA_HEADS * u < n_keys ? ((const uint32_t*)srcs[u])[e] : 0u;
#pragma unroll
                    for (int u = 0; u < PER_WARP; ++u)
                        if (warp + LA_HEADS * u < n_keys) ks[(warp + LA_HEADS * u) * row_words + e] = v[u];
                }
            } else {
                TC* kd = (TC*)ks;
                for (int e = lane; e < width; e += 32) {
                    TC v[PER_WARP];
#pragma unroll
                    for (int u = 0; u < PER_WARP; ++u) v[u] = warp + LA_HEADS * u < n_keys ? srcs[u][e] : from_f32<TC>(0.0f);
#pragma unroll
                    for (int u = 0; u < PER_WARP; ++u)
                        if (warp + LA_HEADS * u < n_keys) kd[(warp + LA_HEADS * u) * row_elems + e] = v[u];
                }
            }
        }
        __syncthreads();
        if (!has_head) continue;
        // scores: lane j, key j
        float s = -INFINITY;
        if (lane < n_keys) {
            const float* qh = qs + warp * width;
            float dot = 0.0f;
            if (packed) {
                const uint32_t* kw = ks + (size_t)lane * row_words;
                float dot2 = 0.0f;
                for (int e = 0; e < width / 2; ++e) {
                    const uint32_t w2 = kw[e];
                    dot = fmaf(qh[2 * e], __uint_as_float(w2 << 16), dot);
                    dot2 = fmaf(qh[2 * e + 1], __uint_as_float(w2 & 0xffff0000u), dot2);
                }
                dot += dot2;
            } else {
                const TC* kr = krow_base + (size_t)lane * row_elems;
                for (int e = 0; e < width; ++e) dot = fmaf(qh[e], to_f32(kr[e]), dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pj = lane < n_keys ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);                      // 0 on the first chunk (m = -inf)
        l = l * corr + warp_sum(pj);
        m = m_new;
        ps[warp * LA_KEYS + lane] = pj;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        if (packed) {
            for (int j = 0; j < n_keys; ++j) {
                const float pw = ps[warp * LA_KEYS + j];
                const uint32_t* kw = ks + (size_t)j * row_words;
#pragma unroll
                for (int i = 0; i < NACC / 2; ++i) {
                    const int e = 2 * lane + 64 * i;
                    if (e < rank) {
                        const uint32_t w2 = kw[lane + 32 * i];
                        acc[2 * i] = fmaf(pw, __uint_as_float(w2 << 16), acc[2 * i]);
                        acc[2 * i + 1] = fmaf(pw, __uint_as_float(w2 & 0xffff0000u), acc[2 * i + 1]);
                    }
                }
            }
        } else {
            for (int j = 0; j < n_keys; ++j) {
                const float pw = ps[warp * LA_KEYS + j];
                const TC* kr = krow_base + (size_t)j * row_elems;
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int e = lane + 32 * i;
                    if (e < rank) acc[i] = fmaf(pw, to_f32(kr[e]), acc[i]);
                }
            }
        }
        __syncwarp();
    }
    if (!has_head) return;
    const size_t item = (size_t)r * heads + head;
    float* pacc = part_acc ? part_acc + (item * gridDim.z + blockIdx.z) * rank : nullptr;
    if (pacc && lane == 0) {
        part_ml[(item * gridDim.z + blockIdx.z) * 2] = m;
        part_ml[(item * gridDim.z + blockIdx.z) * 2 + 1] = l;
    }
    TC* dst = out + ((size_t)head * T + r) * rank;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int e = packed ? 2 * lane + 64 * (i / 2) + (i & 1) : lane + 32 * i;
        if (e < rank) {
            if (pacc) pacc[e] = acc[i];
            else dst[e] = from_f32<TC>(acc[i] * inv);
        }
    }
}

// the stretches of a row's keys, merged in order: out = sum_z e^(m_z - M) acc_z / sum_z e^(m_z - M) l_z
template <typename TC>
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits, int split_keys,
                                    int rank, int heads, int T, const int* __restrict__ positions, TC* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x, head = blockIdx.y;
    const int nz = min(splits, (positions[r] + split_keys) / split_keys);
    const size_t item = (size_t)r * heads + head;
    const float* ml = part_ml + item * splits * 2;
    float M = -INFINITY;
    for (int z = 0; z < nz; ++z) M = fmaxf(M, ml[2 * z]);
    float L = 0.0f;
    for (int z = 0; z < nz; ++z) L += expf(ml[2 * z] - M) * ml[2 * z + 1];
    const float inv = 1.0f / L;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) {
        float v = 0.0f;
        for (int z = 0; z < nz; ++z) v = fmaf(expf(ml[2 * z] - M), part_acc[(item * splits + z) * rank + e], v);
        out[((size_t)head * T + r) * rank + e] = from_f32<TC>(v * inv);
    }
}

template <typename TO>
__global__ void latent_gate_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ld_gate, int heads,
                                       int vdim, int T, TO* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
        const int h = i / vdim, e = i % vdim;
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)r * ld_gate + h])) : 1.0f;
        out[(size_t)r * heads * vdim + i] = from_f32<TO>(o[((size_t)h * T + r) * vdim + e] * g);
    }
}

template <typename TO>
__global__ void latent_q_norm_kernel(const float* __restrict__ x, int ld, int offset, int n, const float* __restrict__ w, float eps,
                                     TO* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float scratch[32];
    const float* src = x + (size_t)blockIdx.x * ld + offset;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) scratch[warp] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < nw; ++i) total += scratch[i];
    const float scale = 1.0f / sqrtf(total / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = from_f32<TO>(src[i] * scale * w[i]);
}

}  // namespace

// out [T, n] = rms(x[:, offset : offset + n]) * w; x float32 with row stride ld
CJ_EXPORT int cj_latent_q_norm(const float* x, int ld, int offset, int n, const float* w, float eps, void* out, int out_dtype, int T,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!x || !w || !out || n <= 0 || offset < 0 || ld < offset + n) return CJ_ERR_ARG;
    const int threads = n >= 1024 ? 256 : 128;
    if (out_dtype == CJ_F32) cj::launch(latent_q_norm_kernel<float>, dim3(T), dim3(threads), 0, stream, x, ld, offset, n, w, eps, (float*)out);
    else if (out_dtype == CJ_BF16) cj::launch(latent_q_norm_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x, ld, offset, n, w, eps, (__nv_bfloat16*)out);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_latent_kv_write(const float* d, int ld, int rank, int rot, int rotary, const float* w, float eps, const float* inv_freq,
                                 const int* positions, const int* row_req, const int* table, int table_stride, int page_tokens,
                                 void* plane, int cache_dtype, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!d || !w || !positions || !row_req || !table || !plane || rank <= 0 || rot < 0 || page_tokens <= 0) return CJ_ERR_ARG;
    if ((rotary & 1) || rotary < 0 || rotary > rot || (rotary > 0 && !inv_freq)) return CJ_ERR_SIZE;
    int threads = rank >= 512 ? 256 : 128;
    if (cache_dtype == CJ_F32) cj::launch(latent_kv_write_kernel<float>, dim3(T), dim3(threads), 0, stream, d, ld, rank, rot, rotary, w, eps, inv_freq, positions, row_req, table, table_stride, page_tokens, (float*)plane);
    else if (cache_dtype == CJ_BF16) cj::launch(latent_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, d, ld, rank, rot, rotary, w, eps, inv_freq, positions, row_req, table, table_stride, page_tokens, (__nv_bfloat16*)plane);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_latent_q_split(const float* q, int ld, int heads, int dim, int rot, int rotary, const float* inv_freq, const int* positions,
                                int T, void* q_plain, int plain_dtype, float* q_rot, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q || !positions || !q_plain || !q_rot || heads <= 0 || dim <= 0 || rot < 0) return CJ_ERR_ARG;
    if ((rotary & 1) || rotary < 0 || rotary > rot || (rotary > 0 && !inv_freq)) return CJ_ERR_SIZE;
    int threads = heads * dim >= 2048 ? 256 : 128;
    if (plain_dtype == CJ_F32) cj::launch(latent_q_split_kernel<float>, dim3(T), dim3(threads), 0, stream, q, ld, heads, dim, rot, rotary, inv_freq, positions, T, (float*)q_plain, q_rot);
    else if (plain_dtype == CJ_BF16) cj::launch(latent_q_split_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, q, ld, heads, dim, rot, rotary, inv_freq, positions, T, (__nv_bfloat16*)q_plain, q_rot);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

// split_keys > 0: a row's keys are cut into stretches of that many (a multiple of 32), one block each;
// part_acc [T, heads, splits, rank] and part_ml [T, heads, splits, 2] (float32) then hold the
// stretches' results, splits = ceil(max_context / split_keys).  split_keys = 0: one block a row.
CJ_EXPORT int cj_latent_attention(const float* q_abs, const float* q_rot, const void* plane, int cache_dtype, int rank, int rot,
                                  int heads, int T, const int* positions, const int* row_req, const int* table, int table_stride,
                                  int page_tokens, float scale, void* out, int split_keys, int splits, float* part_acc,
                                  float* part_ml, const float* sink, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!q_abs || !q_rot || !plane || !positions || !row_req || !table || !out) return CJ_ERR_ARG;
    if (rank <= 0 || rank > 1024 || rot < 0 || heads <= 0 || page_tokens <= 0) return CJ_ERR_SIZE;
    if (split_keys < 0 || split_keys % LA_KEYS != 0 || (split_keys > 0 && (splits < 1 || splits > 65535 || !part_acc || !part_ml))) return CJ_ERR_ARG;
    const int width = rank + rot;
    const int esize = cache_dtype == CJ_F32 ? 4 : 2;
    int row_words = (width * esize + 3) / 4;
    if ((row_words & 1) == 0) row_words += 1;
    const size_t smem = (size_t)LA_HEADS * width * 4 + (size_t)LA_HEADS * LA_KEYS * 4 + (size_t)LA_KEYS * row_words * 4;
    if (smem > 200 * 1024) return CJ_ERR_SIZE;
    dim3 grid(T, (heads + LA_HEADS - 1) / LA_HEADS, split_keys > 0 ? splits : 1);
    if (grid.y > 65535) return CJ_ERR_SIZE;
    const int nacc = (rank + 31) / 32;
    float* pa = split_keys > 0 ? part_acc : nullptr;
    float* pm = split_keys > 0 ? part_ml : nullptr;
#define LAUNCH(TC, N)                                                                                                  \
    do {                                                                                                               \
        static bool sized_##N = false;                                                                                 \
        if (!sized_##N) {                                                                                              \
            cudaFuncSetAttribute(latent_attention_kernel<TC, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            sized_##N = true;                                                                                          \
        }                                                                                                              \
        cj::launch(latent_attention_kernel<TC, N>, grid, dim3(LA_HEADS * 32), smem, stream, q_abs, q_rot, (const TC*)plane, \
                   rank, rot, heads, T, positions, row_req, table, table_stride, page_tokens, scale, (TC*)out, row_words, \
                   split_keys, pa, pm, sink);                                                                          \
        if (split_keys > 0)                                                                                            \
            cj::launch(latent_merge_kernel<TC>, dim3(T, heads), dim3(128), 0, stream, (const float*)pa, (const float*)pm, splits, \
                       split_keys, rank, heads, T, positions, (TC*)out);                                               \
    } while (0)
#define PICK(TC)                                  \
    do {                                          \
        if (nacc <= 4) LAUNCH(TC, 4);             \
        else if (nacc <= 8) LAUNCH(TC, 8);        \
        else if (nacc <= 16) LAUNCH(TC, 16);      \
        else LAUNCH(TC, 32);                      \
    } while (0)
    if (cache_dtype == CJ_F32) PICK(float);
    else if (cache_dtype == CJ_BF16) PICK(__nv_bfloat16);
    else return CJ_ERR_DTYPE;
#undef PICK
#undef LAUNCH
    return launch_status();
}

CJ_EXPORT int cj_latent_gate_out(const float* o, const float* gate, int ld_gate, int heads, int vdim, int T, void* out,
                                 int out_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!o || !out || heads <= 0 || vdim <= 0) return CJ_ERR_ARG;
    int threads = heads * vdim >= 2048 ? 256 : 128;
    if (out_dtype == CJ_F32) cj::launch(latent_gate_out_kernel<float>, dim3(T), dim3(threads), 0, stream, o, gate, ld_gate, heads, vdim, T, (float*)out);
    else if (out_dtype == CJ_BF16) cj::launch(latent_gate_out_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, o, gate, ld_gate, heads, vdim, T, (__nv_bfloat16*)out);
    else return CJ_ERR_DTYPE;
    return launch_status();
}
