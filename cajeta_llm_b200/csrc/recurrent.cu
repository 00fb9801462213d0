// Mixers that carry a fixed-size state per request instead of a growing cache, and the
// row-wise kernels of a block that norms a sublayer's OUTPUT.  Everything that enters a
// recurrence is float32: the state, decays and their logarithms, step sizes, gates, unit
// norms.  A step's rows are laid out request after request; every kernel finds a row's
// request, the request's first row and its state slot in the step's device metadata
// (row_req, req_start, req_slot), so the same launch serves prompt portions of any length
// beside single decoded tokens, and a request that a captured step is filled up with
// (slot -1, no rows) is left alone.
//
//   cast_rows          float32 rows -> the activation dtype (a sublayer reads the stream itself)
//   rmsnorm_add        hs += y / sqrt(mean(y^2) + eps) * w
//   scale_rows_gather  out[slot] = weight[pick] * x[token]  (a mixture whose score multiplies the expert's INPUT)
//   short_conv         causal convolution per channel over time (+ bias, + SiLU) whose first
//                      taps-1 inputs come from the request's state; short_conv_commit then
//                      stores the step's last taps-1 inputs
//   ssd_scan           S_t = exp(-A dt) S_(t-1) + dt B_t x_t^T ;  y_t = S_t^T C_t + D x_t
//   delta_scan         S <- g S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q
//   gla_scan           S_t = diag(alpha_t) S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t   (a decay per state row)
//   mlstm_scan         m_t = max(f + m, i) ; S_t = e^(f + m - m_t) S + e^(i - m_t) k v^T ; n likewise with k alone ;
//                      o = S^T q / (max(|n . q|, e^(-m_t)) + floor)
//   rmsnorm_mix2       out (+)= c (a / rms(a) * wa + b / rms(b) * wb)
//   relu2_rows         max(x, 0)^2 into the activation dtype
//   softcap_rows       x <- cap tanh(x / cap), float32 in place (a head whose logits are capped)
//   gated_group_norm   y * silu(z) (or sigmoid(z)) and RMS over equal parts of a row, in either order
//
// The two scans give a thread one column of the state (one value dimension) for a share of
// its rows: a block is (request, head, tile of columns), a column's rows are dealt to DP
// neighbouring lanes, each holding NPER of them in registers, and a sum over the rows is a
// butterfly over those lanes.  Columns never talk to each other; the block's barriers only
// guard the staging of the tokens' inputs.  The tokens of a request are walked in order, which is what makes the result
// independent of how a prompt was cut: the state after token t is the same sequence of
// float32 operations whether t ended a step or not.
#define CJ_LIB "recurrent"
#include "common.cuh"

using namespace cj;

namespace {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += scratch[i];
    return t;
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    cj::after_predecessor();
    cj::release_successor();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(x[i]);
}

__global__ void rmsnorm_add_kernel(float* __restrict__ hs, const float* __restrict__ y, const float* __restrict__ w, float eps, int H) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float scratch[32];
    const float* src = y + (size_t)blockIdx.x * H;
    float* dst = hs + (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] += src[i] * scale * w[i];
}

template <typename TO>
__global__ void scale_rows_gather_kernel(const float* __restrict__ x, const int* __restrict__ slot_of_pick,
                                         const float* __restrict__ weight, int k, int H, TO* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    const int pick = blockIdx.x;
    const float* src = x + (size_t)(pick / k) * H;
    TO* dst = out + (size_t)slot_of_pick[pick] * H;
    const float wt = weight[pick];
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TO>(wt * src[i]);
}

// ---------------------------------------------------------------------------------
// short convolution over time with the request's last taps-1 inputs as state
// state of a slot: [taps-1][C] float32, oldest first
// ---------------------------------------------------------------------------------
template <typename TO>
__global__ void short_conv_kernel(const float* __restrict__ in, int ld_in, int C, int taps, const float* __restrict__ w,
                                  const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                                  const int* __restrict__ row_req, const int* __restrict__ req_start,
                                  const int* __restrict__ req_slot, TO* __restrict__ out, int ld_out, int act) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    const int req = row_req[r];
    const int t = r - req_start[req];
    const int slot = req_slot[req];
    const float* st = state + (size_t)slot * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = bias ? bias[c] : 0.0f;
        for (int j = taps - 1; j >= 0; --j) {          // oldest input first
            const int src_t = t - j;
            const float v = src_t >= 0 ? in[(size_t)(r - j) * ld_in + c] : st[(size_t)(taps - 1 + src_t) * C + c];
            acc = fmaf(w[(size_t)c * taps + (taps - 1 - j)], v, acc);
        }
        if (act) acc = acc / (1.0f + expf(-acc));
        out[(size_t)r * ld_out + c] = from_f32<TO>(acc);
    }
}

__global__ void short_conv_commit_kernel(const float* __restrict__ in, int ld_in, int C, int taps, float* __restrict__ state,
                                         long long slot_stride, const int* __restrict__ req_start,
                                         const int* __restrict__ req_slot) {
    cj::after_predecessor();
    cj::release_successor();
    const int req = blockIdx.x;
    const int slot = req_slot[req];
    const int first = req_start[req], n = req_start[req + 1] - first;
    if (slot < 0 || n <= 0) return;
    float* st = state + (size_t)slot * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        // ascending k: an entry that is kept moves down from k + n, which is read before it is written
        for (int k = 0; k < taps - 1; ++k) {
            const int src_t = n - (taps - 1) + k;
            st[(size_t)k * C + c] = src_t >= 0 ? in[(size_t)(first + src_t) * ld_in + c] : st[(size_t)(k + n) * C + c];
        }
    }
}

// ---------------------------------------------------------------------------------
// the scans
// ---------------------------------------------------------------------------------
struct ScanArgs {
    const float* x;      // the step's rows after convolution and activation, [T, ld]
    int ld;
    int off_a, off_b, off_v;   // ssd: B, C, x ; delta: q, k, v  (column offsets in x)
    const float* raw;    // the step's rows of the plain projections, [T, ld_raw]
    int ld_raw;
    int off_dt, off_beta;      // ssd: dt ; delta: the decay's input a, beta's input b
    const float* A_log; const float* dt_bias; const float* skip;    // per head (skip: ssd's D)
    float* state; long long slot_stride;     // per slot: the heads' matrices in the scan's own layout, float32
    const int* req_start; const int* req_slot;
    float* out;          // [T, heads * cols]
    int heads, groups, rows, cols;           // rows: state rows (N or key dim); cols: value dim
    float q_scale;
    float c0, c1;        // gla: c0 = 1 / tau ; mlstm: c0 = the gates' cap, c1 = the floor added to the read-out's divisor
};

constexpr int SCAN_SSD = 0, SCAN_DELTA = 1, SCAN_GLA = 2, SCAN_MLSTM = 3;

// log(sigmoid(v)) without overflow on either side
__device__ __forceinline__ float log_sigmoid_f(float v) { return fminf(v, 0.0f) - log1pf(expf(-fabsf(v))); }

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A token's inputs (the two vectors over the state's rows, the block's columns of the value
// vector, the two gate inputs) are staged in shared memory TOK tokens at a time, the next
// TOK in flight (cp.async) while these are walked: a token's step then waits on shared
// memory, not on a round trip to L2.  One staged token: [a | b | v: block's columns | 4 scalars],
// a and b laid out so that a lane's NPER rows (part + DP i) are contiguous: index part * NPER + i.
// What does not depend on the state - the unit norms of q and k, softplus, the decay's
// exponential, beta - is worked out for all staged tokens side by side (a warp a token)
// before they are walked, so that the chain from one token's state to the next is only
// decay, one sum over the rows, the update.  The read-out's sum over the rows, which nothing
// waits for, is carried along with the next token's sum (two independent butterflies side by side).
//
// The state of a (slot, head) is kept in the order the threads hold it: element
// ((tile * NPER + i) * 128 + thread) is row part + DP i of column tile * cols_blk + lcol -
// a layout that depends on the state's shape alone, read and written with full coalescing.
// Nothing else reads the state (a slot is zeroed when it is admitted).
__device__ __forceinline__ float lanes_sum(float v, int first) {
    if (first == 1) return warp_sum(v);                     // a column's rows span the whole warp: unrolled
    for (int o = first; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// MODE 2 (gla) stages a third vector over the state's rows, the decays' inputs (from raw, columns off_dt +
// head * rows), which the scalar phase turns into the decays alpha = sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau).
// MODE 3 (mlstm) keeps, beside a thread's share of its column, the same share of the vector n (every column of
// a tile holds it: what a block reads at its start no other block writes) and the running maximum m:
// a (slot, head, tile) holds [S: NPER x 128 | n: NPER x 128 | m: 128] floats.
template <int NPER, int MODE>
__global__ void __launch_bounds__(128) scan_kernel(ScanArgs p, int DP, int TOK) {
    constexpr bool DELTA = MODE == SCAN_DELTA;
    constexpr int NVEC = MODE == SCAN_GLA ? 3 : 2;
    constexpr int TILE_FLOATS = MODE == SCAN_MLSTM ? (2 * NPER + 1) * 128 : NPER * 128;
    cj::after_predecessor();
    cj::release_successor();
    extern __shared__ __align__(16) float staged[];
    const int req = blockIdx.x, head = blockIdx.y;
    const int slot = p.req_slot[req];
    const int first = p.req_start[req], n = p.req_start[req + 1] - first;
    if (slot < 0 || n <= 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cols_per_warp = 32 / DP, cols_blk = 4 * cols_per_warp;
    const int part = lane / cols_per_warp;                  // which share of the state's rows
    const int col0 = blockIdx.z * cols_blk;
    const int lcol = warp * cols_per_warp + (lane % cols_per_warp);
    const int col = col0 + lcol;
    const bool live = col < p.cols;
    const int rows = p.rows, padded = DP * NPER;            // rows rounded up to what the lanes hold
    const int group = head / (p.heads / p.groups);
    const int tail = NVEC * padded + cols_blk;              // where a staged token's four scalars begin
    const int stride = tail + 4;
    float* S = p.state + (size_t)slot * p.slot_stride + ((size_t)head * gridDim.z + blockIdx.z) * TILE_FLOATS;

    // Where a staged token's entries come from is the same for every token: a thread works out, once,
    // the source of the entries it copies (entry e = thread + 128 k) as an offset into the token's row
    // of x (kind 1) or of raw (kind 2), or nothing (kind 0: padding, written as zero).
    constexpr int OWN = 4;                                  // entries a thread remembers; longer tokens take the general loop
    int own_off[OWN], own_kind[OWN];
    auto source = [&](int e, int& off) -> int {
        if (e < NVEC * padded) {
            const int which = e / padded;
            const int v = e - which * padded;               // index part * NPER + i  ->  row part + DP i
            const int d = (v / NPER) + DP * (v % NPER);
            if (which == 2) {                               // gla: the decays' inputs, a row of raw per head
                off = p.off_dt + head * rows + d;
                return d < rows ? 2 : 0;
            }
            off = (which == 0 ? p.off_a : p.off_b) + group * rows + d;
            return d < rows ? 1 : 0;
        }
        if (e < tail) {
            const int c = col0 + e - NVEC * padded;
            off = p.off_v + head * p.cols + c;
            return c < p.cols ? 1 : 0;
        }
        if (MODE != SCAN_GLA && e == tail) { off = p.off_dt + head; return 2; }
        if ((DELTA || MODE == SCAN_MLSTM) && e == tail + 1) { off = p.off_beta + head; return 2; }
        off = 0;
        return 0;
    };
#pragma unroll
    for (int k = 0; k < OWN; ++k) {
        const int e = threadIdx.x + 128 * k;
        own_kind[k] = e < stride ? source(e, own_off[k]) : -1;
        if (e >= stride) own_off[k] = 0;
    }
    auto stage = [&](int chunk, float* buf) {
        const int t0 = chunk * TOK, nt = min(TOK, n - t0);
        for (int tt = 0; tt < nt; ++tt) {
            const size_t row = (size_t)(first + t0 + tt);
            const float* xr = p.x + row * p.ld;
            const float* rr = p.raw + row * p.ld_raw;
            float* dst = buf + tt * stride;
#pragma unroll
            for (int k = 0; k < OWN; ++k) {
                const int e = threadIdx.x + 128 * k;
                if (own_kind[k] > 0) cp_async4(dst + e, (own_kind[k] == 1 ? xr : rr) + own_off[k]);
                else if (own_kind[k] == 0) dst[e] = 0.0f;
            }
            for (int e = threadIdx.x + 128 * OWN; e < stride; e += 128) {
                int off;
                const int kind = source(e, off);
                if (kind > 0) cp_async4(dst + e, (kind == 1 ? xr : rr) + off);
                else dst[e] = 0.0f;
            }
        }
    };

    const int chunks = (n + TOK - 1) / TOK;
    stage(0, staged);
    cp_async_commit();
    float s[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) s[i] = S[i * 128 + threadIdx.x];
    // ssd, delta: A = exp(A_log), bias = the step size's; mlstm: A = the forget gate's bias, bias = the input gate's
    const float A = MODE == SCAN_GLA ? 0.0f : (MODE == SCAN_MLSTM ? p.A_log[head] : expf(p.A_log[head]));
    const float bias = MODE == SCAN_GLA ? 0.0f : p.dt_bias[head];
    const float skip = MODE == SCAN_SSD ? p.skip[head] : 0.0f;
    float nvec[MODE == SCAN_MLSTM ? NPER : 1];
    float m_run = 0.0f;
    if (MODE == SCAN_MLSTM) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) nvec[i] = S[(NPER + i) * 128 + threadIdx.x];
        m_run = S[2 * NPER * 128 + threadIdx.x];
    }
    float* out = p.out + (size_t)first * p.heads * p.cols + head * p.cols + col;
    const size_t out_ld = (size_t)p.heads * p.cols;
    const bool writer = live && part == 0;
    float y_prev = 0.0f;                                    // the token before's read-out, its sum over the lanes still owed
    int t_prev = -1;
    for (int chunk = 0; chunk < chunks; ++chunk) {
        float* cur = staged + (chunk & 1) * TOK * stride;
        if (chunk + 1 < chunks) stage(chunk + 1, staged + ((chunk + 1) & 1) * TOK * stride);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int nt = min(TOK, n - chunk * TOK);
        // the staged tokens' scalars: a warp a token
        for (int tt = warp; tt < nt; tt += 4) {
            float* tk = cur + tt * stride;
            if (DELTA) {
                float qq = 0.0f, kk = 0.0f;
                for (int d = lane; d < padded; d += 32) {
                    qq = fmaf(tk[d], tk[d], qq);
                    kk = fmaf(tk[padded + d], tk[padded + d], kk);
                }
                qq = warp_sum(qq);
                kk = warp_sum(kk);
                if (lane == 0) {
                    const float g0 = tk[tail], g1 = tk[tail + 1];
                    tk[tail] = expf(-A * softplus_f(g0 + bias));          // the decay
                    tk[tail + 1] = sigmoid_f(g1);                         // beta
                    tk[tail + 2] = p.q_scale / sqrtf(qq + 1e-6f);         // q becomes a unit vector times q_scale
                    tk[tail + 3] = 1.0f / sqrtf(kk + 1e-6f);              // k a unit vector
                }
            } else if (MODE == SCAN_GLA) {
                for (int d = lane; d < padded; d += 32) tk[2 * padded + d] = expf(log_sigmoid_f(tk[2 * padded + d]) * p.c0);
            } else if (MODE == SCAN_MLSTM) {
                if (lane == 0) {
                    const float cap = p.c0;
                    tk[tail] = cap * tanhf((tk[tail] + bias) / cap);                          // log of the input gate
                    tk[tail + 1] = log_sigmoid_f(cap * tanhf((tk[tail + 1] + A) / cap));      // log of the forget gate
                }
            } else if (lane == 0) {
                const float dt = softplus_f(tk[tail] + bias);
                tk[tail] = dt;
                tk[tail + 1] = expf(-A * dt);
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* tk = cur + tt * stride;
            const float xv = tk[NVEC * padded + lcol];
            float a[NPER], b[NPER];
            if (NPER % 4 == 0) {
#pragma unroll
                for (int i = 0; i < NPER; i += 4) {
                    const float4 va = *(const float4*)(tk + part * NPER + i);
                    const float4 vb = *(const float4*)(tk + padded + part * NPER + i);
                    a[i] = va.x; a[i + 1] = va.y; a[i + 2] = va.z; a[i + 3] = va.w;
                    b[i] = vb.x; b[i + 1] = vb.y; b[i + 2] = vb.z; b[i + 3] = vb.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    a[i] = tk[part * NPER + i];
                    b[i] = tk[padded + part * NPER + i];
                }
            }
            if (DELTA) {
                const float decay = tk[tail], beta = tk[tail + 1], qs = tk[tail + 2], ks = tk[tail + 3];
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    b[i] *= ks;
                    s[i] *= decay;
                    dot = fmaf(s[i], b[i], dot);
                }
                // this token's S^T k and the token before's read-out: two sums over the lanes, side by side
                if (cols_per_warp == 1) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        dot += __shfl_xor_sync(0xffffffffu, dot, o);
                        y_prev += __shfl_xor_sync(0xffffffffu, y_prev, o);
                    }
                } else {
                    for (int o = cols_per_warp; o < 32; o <<= 1) {
                        dot += __shfl_xor_sync(0xffffffffu, dot, o);
                        y_prev += __shfl_xor_sync(0xffffffffu, y_prev, o);
                    }
                }
                if (writer && t_prev >= 0) out[(size_t)t_prev * out_ld] = y_prev;
                const float u = beta * (xv - dot);
                float y = 0.0f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    s[i] = fmaf(b[i], u, s[i]);
                    y = fmaf(s[i], a[i] * qs, y);
                }
                y_prev = y;
                t_prev = chunk * TOK + tt;
            } else if (MODE == SCAN_GLA) {
                // a = q, b = k, a row's decay from the third staged vector
                float y = 0.0f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    s[i] = fmaf(tk[2 * padded + part * NPER + i], s[i], b[i] * xv);
                    y = fmaf(s[i], a[i] * p.q_scale, y);
                }
                y = lanes_sum(y, cols_per_warp);
                if (writer) out[(size_t)(chunk * TOK + tt) * out_ld] = y;
            } else if (MODE == SCAN_MLSTM) {
                const float li = tk[tail], lf = tk[tail + 1];
                const float m_new = fmaxf(lf + m_run, li);
                const float keep = expf(lf + m_run - m_new), take = expf(li - m_new);
                m_run = m_new;
                float y = 0.0f, nq = 0.0f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    const float kb = take * b[i], qa = a[i] * p.q_scale;
                    s[i] = fmaf(keep, s[i], kb * xv);
                    nvec[i] = fmaf(keep, nvec[i], kb);
                    y = fmaf(s[i], qa, y);
                    nq = fmaf(nvec[i], qa, nq);
                }
                if (cols_per_warp == 1) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        y += __shfl_xor_sync(0xffffffffu, y, o);
                        nq += __shfl_xor_sync(0xffffffffu, nq, o);
                    }
                } else {
                    for (int o = cols_per_warp; o < 32; o <<= 1) {
                        y += __shfl_xor_sync(0xffffffffu, y, o);
                        nq += __shfl_xor_sync(0xffffffffu, nq, o);
                    }
                }
                if (writer) out[(size_t)(chunk * TOK + tt) * out_ld] = y / (fmaxf(fabsf(nq), expf(-m_run)) + p.c1);
            } else {
                // a = B, b = C
                const float dt = tk[tail], decay = tk[tail + 1];
                const float dx = dt * xv;
                float y = 0.0f;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    s[i] = fmaf(decay, s[i], a[i] * dx);
                    y = fmaf(s[i], b[i], y);
                }
                y = lanes_sum(y, cols_per_warp);
                if (writer) out[(size_t)(chunk * TOK + tt) * out_ld] = fmaf(skip, xv, y);
            }
        }
        __syncthreads();                       // everyone has walked this buffer before it is staged into again
    }
    if (DELTA) {
        y_prev = lanes_sum(y_prev, cols_per_warp);
        if (writer && t_prev >= 0) out[(size_t)t_prev * out_ld] = y_prev;
    }
#pragma unroll
    for (int i = 0; i < NPER; ++i) S[i * 128 + threadIdx.x] = s[i];
    if (MODE == SCAN_MLSTM) {
#pragma unroll
        for (int i = 0; i < NPER; ++i) S[(NPER + i) * 128 + threadIdx.x] = nvec[i];
        S[2 * NPER * 128 + threadIdx.x] = m_run;
    }
}

// ---------------------------------------------------------------------------------
// y * silu(z) and an RMS over equal parts of the row, in either order:
//   gate_first:  v = y * silu(z);  out = v / rms_part(v) * w
//   else:        out = y / rms_part(y) * w * silu(z)
// (bit 0 of `gate_first` is the order; bit 1 set: the gate is sigmoid(z) instead of silu(z))
// w has w_len entries and is indexed by (column % w_len): a weight per column of the row,
// or one shared by all parts.  One warp per part.
// ---------------------------------------------------------------------------------
template <typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int n, int part_len, const float* __restrict__ z, int ld_z,
                                        const float* __restrict__ w, int w_len, float eps, int gate_first,
                                        TO* __restrict__ out) {
    cj::after_predecessor();
    cj::release_successor();
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int parts = n / part_len;
    const bool plain_sigmoid = (gate_first & 2) != 0;
    gate_first &= 1;
    for (int g = blockIdx.y * nw + warp; g < parts; g += gridDim.y * nw) {
        const float* yr = y + (size_t)r * n + (size_t)g * part_len;
        const float* zr = z + (size_t)r * ld_z + (size_t)g * part_len;
        float ss = 0.0f;
        for (int i = lane; i < part_len; i += 32) {
            float v = yr[i];
            if (gate_first) { const float zz = zr[i]; v *= (plain_sigmoid ? 1.0f : zz) / (1.0f + expf(-zz)); }
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)part_len + eps);
        for (int i = lane; i < part_len; i += 32) {
            const float zz = zr[i];
            const float gate = (plain_sigmoid ? 1.0f : zz) / (1.0f + expf(-zz));
            const int c = g * part_len + i;
            float v = yr[i];
            v = gate_first ? (v * gate) * scale * w[c % w_len] : v * scale * w[c % w_len] * gate;
            out[(size_t)r * n + c] = from_f32<TO>(v);
        }
    }
}

// out (+)= c (a / rms(a) * wa + b / rms(b) * wb): the results of two mixers that read the same input, each
// RMS-normed over the row with a weight of its own, averaged (c = 1/2) or summed.  A block a row.
__global__ void rmsnorm_mix2_kernel(const float* __restrict__ a, const float* __restrict__ wa, const float* __restrict__ b,
                                    const float* __restrict__ wb, float eps, float c, int accumulate, float* __restrict__ out, int H) {
    cj::after_predecessor();
    cj::release_successor();
    __shared__ float scratch[32];
    const float* ra = a + (size_t)blockIdx.x * H;
    const float* rb = b + (size_t)blockIdx.x * H;
    float* dst = out + (size_t)blockIdx.x * H;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        sa = fmaf(ra[i], ra[i], sa);
        sb = fmaf(rb[i], rb[i], sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float fa = 1.0f / sqrtf(sa / (float)H + eps), fb = 1.0f / sqrtf(sb / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = c * (ra[i] * fa * wa[i] + rb[i] * fb * wb[i]);
        dst[i] = accumulate ? dst[i] + v : v;
    }
}

// max(x, 0)^2 into the activation dtype (the activation of an ungated expert whose product was stored in float32)
template <typename TO>
__global__ void relu2_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, long long n) {
    cj::after_predecessor();
    cj::release_successor();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(x[i], 0.0f);
        out[i] = from_f32<TO>(v * v);
    }
}

// x <- cap tanh(x / cap), in place, float32
__global__ void softcap_rows_kernel(float* __restrict__ x, float cap, long long n) {
    cj::after_predecessor();
    cj::release_successor();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace

// Lanes a column's rows are dealt to (4, 8, 16 or 32).  Every (column, token) costs a warp its staging,
// its butterflies and its store whatever the lanes hold, so fewer lanes a column - more columns a
// warp - mean fewer instructions in all; but one request's scan is a chain, and with too few warps
// the chain's latencies lie bare.  So: the fewest lanes (at least 8 where there are 8 rows) that
// still give ONE request's scan a warp for each of a B200's 592 warp schedulers; and few enough rows
// a lane (64) to stay in registers.  Measured on two scans of a 2,048-token prompt, 8 / 16 / 32 lanes:
// 32 + 8 heads 2.40 / 2.46 / 2.36 ms (all short of warps), 64 + 16 heads 2.63 / 2.85 / 3.64 ms.
// The state's layout follows from this number, so it depends on the state's shape alone.
static int scan_lanes(int heads, int rows, int cols) {
    int dp = 4;
    while (dp < 32 && dp < rows && (dp < 8 || (long long)heads * cols * dp / 32 < 592)) dp <<= 1;
    while (dp < 32 && (rows + dp - 1) / dp > 64) dp <<= 1;
    return dp;
}

CJ_EXPORT int cj_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!x || !out) return CJ_ERR_ARG;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == CJ_F32) cj::launch(cast_rows_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (float*)out, n);
    else if (out_dtype == CJ_BF16) cj::launch(cast_rows_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, n);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_rmsnorm_add(float* hs, const float* y, const float* w, float eps, int rows, int H, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!hs || !y || !w || H <= 0) return CJ_ERR_ARG;
    int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    cj::launch(rmsnorm_add_kernel, dim3(rows), dim3(threads), 0, stream, hs, y, w, eps, H);
    return launch_status();
}

CJ_EXPORT int cj_scale_rows_gather(const float* x, const int* slot_of_pick, const float* weight, int picks, int k, int H,
                                   void* out, int out_dtype, cudaStream_t stream) {
    if (picks <= 0) return 0;
    if (!x || !slot_of_pick || !weight || !out || k < 1 || H <= 0) return CJ_ERR_ARG;
    int threads = H >= 1024 ? 256 : 128;
    if (out_dtype == CJ_F32) cj::launch(scale_rows_gather_kernel<float>, dim3(picks), dim3(threads), 0, stream, x, slot_of_pick, weight, k, H, (float*)out);
    else if (out_dtype == CJ_BF16) cj::launch(scale_rows_gather_kernel<__nv_bfloat16>, dim3(picks), dim3(threads), 0, stream, x, slot_of_pick, weight, k, H, (__nv_bfloat16*)out);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_short_conv(const float* in, int ld_in, int C, int taps, const float* w, const float* bias, const float* state,
                            long long slot_stride, const int* row_req, const int* req_start, const int* req_slot, void* out,
                            int ld_out, int out_dtype, int act, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!in || !w || !state || !row_req || !req_start || !req_slot || !out || C <= 0 || taps < 1) return CJ_ERR_ARG;
    int threads = C >= 512 ? 256 : 128;
    int by = (C + threads - 1) / threads;
    if (by > 64) by = 64;
    dim3 grid(T, by);
    if (out_dtype == CJ_F32) cj::launch(short_conv_kernel<float>, grid, dim3(threads), 0, stream, in, ld_in, C, taps, w, bias, state, slot_stride, row_req, req_start, req_slot, (float*)out, ld_out, act);
    else if (out_dtype == CJ_BF16) cj::launch(short_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, in, ld_in, C, taps, w, bias, state, slot_stride, row_req, req_start, req_slot, (__nv_bfloat16*)out, ld_out, act);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_short_conv_commit(const float* in, int ld_in, int C, int taps, float* state, long long slot_stride,
                                   const int* req_start, const int* req_slot, int requests, cudaStream_t stream) {
    if (requests <= 0 || taps <= 1) return 0;
    if (!in || !state || !req_start || !req_slot || C <= 0) return CJ_ERR_ARG;
    int threads = C >= 512 ? 256 : 128;
    int by = (C + threads - 1) / threads;
    if (by > 64) by = 64;
    cj::launch(short_conv_commit_kernel, dim3(requests, by), dim3(threads), 0, stream, in, ld_in, C, taps, state, slot_stride, req_start, req_slot);
    return launch_status();
}

// mode 0: the state-space scan (off_a = B, off_b = C, off_v = x; off_dt in raw);
// mode 1: the gated delta rule (off_a = q, off_b = k, off_v = v; off_dt = decay input, off_beta in raw);
// mode 2: gated linear attention (off_a = q, off_b = k, off_v = v; raw columns off_dt + head * rows + d = the decays'
//         inputs; c0 = 1 / tau; A_log, dt_bias unused);
// mode 3: the matrix memory with exponential gating (off_a = q, off_b = k, off_v = v; raw columns off_dt + head = the
//         input gate's, off_beta + head = the forget gate's pre-activation; dt_bias = the input gate's bias, A_log = the
//         forget gate's; c0 = the gates' cap, c1 = the floor added to the read-out's divisor).
static long long scan_tile_floats(int mode, int nper) { return mode == 3 ? (long long)(2 * nper + 1) * 128 : (long long)nper * 128; }

CJ_EXPORT int cj_state_scan(int mode, const float* x, int ld, int off_a, int off_b, int off_v, const float* raw, int ld_raw,
                            int off_dt, int off_beta, const float* A_log, const float* dt_bias, const float* skip, float* state,
                            long long slot_stride, long long state_floats, const int* req_start, const int* req_slot, float* out,
                            int requests, int heads, int groups, int rows, int cols, float q_scale, float c0, float c1,
                            cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (mode < 0 || mode > 3) return CJ_ERR_ARG;
    if (!x || !raw || !state || !req_start || !req_slot || !out) return CJ_ERR_ARG;
    if (mode != 2 && (!A_log || !dt_bias)) return CJ_ERR_ARG;
    if (mode == 0 && !skip) return CJ_ERR_ARG;
    if ((mode == 2 || mode == 3) && !(c0 > 0.0f)) return CJ_ERR_ARG;
    if (heads <= 0 || groups <= 0 || heads % groups != 0 || rows <= 0 || cols <= 0) return CJ_ERR_SIZE;
    const int DP = scan_lanes(heads, rows, cols);
    const int per = (rows + DP - 1) / DP;
    if (per > 64) return CJ_ERR_SIZE;
    int nper = 1;
    while (nper < per) nper <<= 1;
    ScanArgs p{x, ld, off_a, off_b, off_v, raw, ld_raw, off_dt, off_beta, A_log, dt_bias, skip, state, slot_stride,
               req_start, req_slot, out, heads, groups, rows, cols, q_scale, c0, c1};
    const int cols_per_block = 4 * (32 / DP);
    dim3 grid(requests, heads, (cols + cols_per_block - 1) / cols_per_block);
    if (grid.y > 65535 || grid.z > 65535) return CJ_ERR_SIZE;
    if (state_floats < (long long)heads * grid.z * scan_tile_floats(mode, nper)) return CJ_ERR_SIZE;
    // tokens staged at a time: up to 16, as many as 96 KB of shared memory hold twice
    const size_t token_bytes = (size_t)((mode == 2 ? 3 : 2) * DP * nper + cols_per_block + 4) * sizeof(float);
    int TOK = (int)((96 * 1024) / (2 * token_bytes));
    if (TOK > 16) TOK = 16;
    if (TOK < 1) return CJ_ERR_SIZE;
    const size_t smem = 2 * (size_t)TOK * token_bytes;
#define LAUNCH_MODE(N, M)                                                                                               \
    do {                                                                                                                \
        static bool sized = false;                                                                                      \
        if (!sized) {                                                                                                   \
            cudaFuncSetAttribute(scan_kernel<N, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);            \
            sized = true;                                                                                               \
        }                                                                                                               \
        cj::launch(scan_kernel<N, M>, grid, dim3(128), smem, stream, p, DP, TOK);                                       \
    } while (0)
#define LAUNCH(N)                                                                                                       \
    do {                                                                                                                \
        if (mode == 0) LAUNCH_MODE(N, SCAN_SSD);                                                                        \
        else if (mode == 1) LAUNCH_MODE(N, SCAN_DELTA);                                                                 \
        else if (mode == 2) LAUNCH_MODE(N, SCAN_GLA);                                                                   \
        else LAUNCH_MODE(N, SCAN_MLSTM);                                                                                \
    } while (0)
    switch (nper) {
        case 1: LAUNCH(1); break;
        case 2: LAUNCH(2); break;
        case 4: LAUNCH(4); break;
        case 8: LAUNCH(8); break;
        case 16: LAUNCH(16); break;
        case 32: LAUNCH(32); break;
        default: LAUNCH(64);
    }
#undef LAUNCH
#undef LAUNCH_MODE
    return launch_status();
}

// floats of state one (slot, schedule entry) needs for heads matrices of rows x cols in the scan's own layout
// (mode 3 keeps a vector over the rows and a scalar beside every tile of a matrix)
CJ_EXPORT long long cj_state_scan_floats_mode(int mode, int heads, int rows, int cols) {
    if (heads <= 0 || rows <= 0 || cols <= 0) return 0;
    const int DP = scan_lanes(heads, rows, cols);
    const int per = (rows + DP - 1) / DP;
    int nper = 1;
    while (nper < per) nper <<= 1;
    const int cols_per_block = 4 * (32 / DP);
    return (long long)heads * ((cols + cols_per_block - 1) / cols_per_block) * scan_tile_floats(mode, nper);
}

CJ_EXPORT long long cj_state_scan_floats(int heads, int rows, int cols) { return cj_state_scan_floats_mode(0, heads, rows, cols); }

CJ_EXPORT int cj_gated_group_norm(const float* y, int n, int part_len, const float* z, int ld_z, const float* w, int w_len,
                                  float eps, int gate_first, void* out, int out_dtype, int rows, cudaStream_t stream) {
    // gate_first: bit 0 the gate multiplies before the norm's statistics, bit 1 the gate is sigmoid(z), not silu(z)
    if (rows <= 0) return 0;
    if (!y || !z || !w || !out || n <= 0 || part_len <= 0 || w_len <= 0) return CJ_ERR_ARG;
    if (n % part_len != 0) return CJ_ERR_SIZE;
    const int parts = n / part_len;
    int warps = parts < 8 ? parts : 8;
    int by = (parts + warps - 1) / warps;
    if (by > 64) by = 64;
    dim3 grid(rows, by);
    if (out_dtype == CJ_F32) cj::launch(gated_group_norm_kernel<float>, grid, dim3(warps * 32), 0, stream, y, n, part_len, z, ld_z, w, w_len, eps, gate_first, (float*)out);
    else if (out_dtype == CJ_BF16) cj::launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream, y, n, part_len, z, ld_z, w, w_len, eps, gate_first, (__nv_bfloat16*)out);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_rmsnorm_mix2(const float* a, const float* wa, const float* b, const float* wb, float eps, float c, int accumulate,
                              float* out, int rows, int H, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!a || !wa || !b || !wb || !out || H <= 0) return CJ_ERR_ARG;
    int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    cj::launch(rmsnorm_mix2_kernel, dim3(rows), dim3(threads), 0, stream, a, wa, b, wb, eps, c, accumulate, out, H);
    return launch_status();
}

CJ_EXPORT int cj_relu2_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!x || !out) return CJ_ERR_ARG;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == CJ_F32) cj::launch(relu2_rows_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (float*)out, n);
    else if (out_dtype == CJ_BF16) cj::launch(relu2_rows_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, n);
    else return CJ_ERR_DTYPE;
    return launch_status();
}

CJ_EXPORT int cj_softcap_rows(float* x, float cap, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!x || !(cap > 0.0f)) return CJ_ERR_ARG;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cj::launch(softcap_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, cap, n);
    return launch_status();
}
