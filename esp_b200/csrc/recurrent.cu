// Layers with a recurrent state of fixed size per sequence.
//
//  * token shift: every row is mixed with the row before it in its sequence (the last row of the step before comes
//    from the sequence's state), once per consumer, each with a mixing vector of its own;
//  * the gated outer-product recurrence that linear-attention layers share,
//        S_t = diag(d_t) S_(t-1) + k_t v_t^T          S: [K, V] per head, 32-bit, one per sequence
//        o_t = (S_(t-1) or S_t, + diag(b) k_t v_t^T)^T q_t
//    with the gates made from the projections' raw outputs as the rows are staged (so that decays, their
//    exponentials and the sigmoid never leave 32-bit);
//  * the per-head RMS norm of the recurrence's output with an optional SiLU gate.
//
// The recurrence is sequential in t by definition and everything that enters it is 32-bit, so it runs on the CUDA
// cores: a block owns (sequence, head, a tile of value columns), a thread a value column and a slice of the key
// channels, which it keeps in registers for the whole run of tokens.  Tokens are staged CHUNK at a time through two
// shared-memory buffers filled by cp.async, so the loop over tokens never waits for global memory; inside a chunk no
// block-wide barrier is needed (the key slices of a column sit in neighbouring lanes and are added by shuffles).
// The order of every addition depends on the token and the channel alone: cutting a sequence into steps, or
// batching it with others, changes no bit.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------- token shift
// out[m, n, :] = h[n] + (prev(n) - h[n]) * mu[m];  prev(n) = h[n - 1] within the step's run of the sequence, or the
// sequence's state row for the run's first token (zeros for a sequence's first token: a fresh slot is zeroed).
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ prev_state, long long state_stride,
                                       const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                       const int* __restrict__ seq_slot, const float* __restrict__ mu, T* __restrict__ out,
                                       int n_mix, int n_rows, int width) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n];
    const bool first = n == seq_start[seq];
    const float* ps = prev_state + (size_t)seq_slot[seq] * state_stride;
    const T* cur = h + (size_t)n * width;
    const T* before = h + (size_t)(n - 1) * width;
    if (sizeof(T) == 2 && width % 8 == 0 && ((size_t)h % 16) == 0 && ((size_t)out % 16) == 0 && state_stride % 4 == 0 &&
        ((size_t)prev_state % 16) == 0) {
        // eight channels a thread: one 16-byte load of the row (and of the row before), one 16-byte store per mix
        for (int d = threadIdx.x * 8; d < width; d += blockDim.x * 8) {
            float c[8], p[8];
            const uint4 cv = *reinterpret_cast<const uint4*>(cur + d);
            const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cv);
#pragma unroll
            for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(c2[i]); c[2 * i] = f.x; c[2 * i + 1] = f.y; }
            if (first) {
                const float4 a = *reinterpret_cast<const float4*>(ps + d), b = *reinterpret_cast<const float4*>(ps + d + 4);
                p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w; p[4] = b.x; p[5] = b.y; p[6] = b.z; p[7] = b.w;
            } else {
                const uint4 pv = *reinterpret_cast<const uint4*>(before + d);
                const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
                for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(p2[i]); p[2 * i] = f.x; p[2 * i + 1] = f.y; }
            }
            for (int m = 0; m < n_mix; m++) {
                const float* mm = mu + (size_t)m * width + d;
                uint4 o;
                unsigned* o1 = reinterpret_cast<unsigned*>(&o);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(fmaf(p[2 * i] - c[2 * i], mm[2 * i], c[2 * i]),
                                                             fmaf(p[2 * i + 1] - c[2 * i + 1], mm[2 * i + 1], c[2 * i + 1]));
                    o1[i] = *reinterpret_cast<unsigned*>(&v);
                }
                *reinterpret_cast<uint4*>(out + ((size_t)m * n_rows + n) * width + d) = o;
            }
        }
        return;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        const float c = to_f32(cur[d]);
        const float p = first ? ps[d] : to_f32(before[d]);
        const float diff = p - c;
        for (int m = 0; m < n_mix; m++)
            out[((size_t)m * n_rows + n) * width + d] = from_f32<T>(fmaf(diff, mu[(size_t)m * width + d], c));
    }
}

// state row of every sequence <- its last row of the step
template <typename T>
__global__ void token_shift_keep_kernel(const T* __restrict__ h, float* __restrict__ prev_state, long long state_stride,
                                        const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int width) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int last = seq_start[b + 1] - 1;
    if (last < seq_start[b]) return;
    float* ps = prev_state + (size_t)seq_slot[b] * state_stride;
    for (int d = threadIdx.x; d < width; d += blockDim.x) ps[d] = to_f32(h[(size_t)last * width + d]);
}

// ---------------------------------------------------------------------------------------------- the recurrence
constexpr int SCAN_THREADS = 128;
// Tiling constants that were measured against each other (2,048 tokens of one sequence, 16 heads of 128 x 128, and
// eight such sequences): columns per thread 1 / 2 / 4: 588 / 793 / 1,258 us and 2,464 / 1,862 / 1,540 us; blocks of 64
// threads for short grids: 627 us; no unrolling of the token loop: 625 us.  The defaults serve the single long prompt.
#ifndef ESP_SCAN_CPT
#define ESP_SCAN_CPT 1
#endif
#ifndef ESP_SCAN_SMALL_THREADS
#define ESP_SCAN_SMALL_THREADS 128
#endif
#ifndef ESP_SCAN_UNROLL
#define ESP_SCAN_UNROLL 4
#endif
constexpr int SCAN_UNROLL = ESP_SCAN_UNROLL;
constexpr int CPT = ESP_SCAN_CPT;   // value columns a thread keeps: a token's q, k, d are read once for all of them
constexpr int KT = 16;          // key channels a thread keeps
constexpr int KTP = KT + 4;     // a slice's stride in shared memory: slices 80 bytes apart fall into different banks
constexpr int CHUNK = 16;       // tokens staged at a time
constexpr int MAX_K = 16 * KT;  // key channels of a head that the kernel takes

enum : int {
    GATE_EXP_EXP = 0,       // d = exp(-exp(g + bias));  k, q as given;  o reads S_(t-1) + diag(bonus) k v^T
    GATE_LOWER_SIGMOID = 1, // d = lower + (1 - lower) * sigmoid(g + bias);  k = 1 - d;  q = silu(q);  o reads S_t
    GATE_SCALAR = 2         // d is one number per head and token, ready made (g: [rows, H]);  k, q as given;  o reads S_t
};

// The gates, written with explicit operations so that the kernel that makes them ahead of the recurrence and the
// recurrence itself (when it makes them as it stages rows) give the same bits.
__device__ __forceinline__ float gate_decay(float raw) { return expf(-expf(raw)); }
__device__ __forceinline__ float gate_sigmoid(float raw) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-raw))); }
__device__ __forceinline__ float gate_lower(float raw, float lo) { return __fmaf_rn(__fsub_rn(1.0f, lo), gate_sigmoid(raw), lo); }
__device__ __forceinline__ float gate_silu(float z) { return __fmul_rn(z, gate_sigmoid(z)); }

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// q, k, g: [rows, ld*] float (k may be null in GATE_LOWER_SIGMOID); v: [rows, ldv]; head h reads columns
// [h*K, (h+1)*K) (v: [h*V, (h+1)*V)).  state: [slots, state_stride] floats, the head's block at h*V*K laid out
// [V][K] (a thread's key slice is contiguous).  out: [rows, H*V] float.
template <int MODE, bool READY>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_scan_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                  const float* __restrict__ g, long long ldg, const float* __restrict__ v, long long ldv,
                  const float* __restrict__ gate_bias, const float* __restrict__ lower, const float* __restrict__ bonus,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, float* __restrict__ out, int H, int K, int V, int ks, int vt) {
    pdl_trigger();
    extern __shared__ __align__(16) float smem[];
    const int kp = ks * KTP;                       // floats of one token's q (or k, or d): the threads' slices, padded
    auto at = [](int c) { return (c / KT) * KTP + (c % KT); };     // where key channel c lies in such a row
    // per buffer: q[CHUNK][kp], k[CHUNK][kp], d[CHUNK][kp], v[CHUNK][vt]
    const int buf_floats = CHUNK * (3 * kp + vt);
    const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * vt;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int part = tid % ks, col = (tid / ks) * CPT;   // neighbouring lanes hold the slices of one pair of columns
    const int vcol = v0 + col;
    bool live[CPT];
#pragma unroll
    for (int j = 0; j < CPT; j++) live[j] = col + j < vt && vcol + j < V;
    const int row0 = seq_start[b], row1 = seq_start[b + 1];
    if (row1 <= row0) return;
    float* srow = state + (size_t)seq_slot[b] * state_stride + ((size_t)h * V + vcol) * K + part * KT;   // column j: + j * K

    // constants of the head: bias / lower bound / bonus per key channel
    __shared__ float c_bias[MAX_K], c_lower[MAX_K], c_bonus[MAX_K];
    for (int i = tid; i < ks * KT; i += nthreads) {
        const bool in = i < K;
        c_bias[i] = in && gate_bias ? gate_bias[h * K + i] : 0.f;
        c_lower[i] = in && lower ? lower[h * K + i] : 0.f;
        c_bonus[i] = in && bonus ? bonus[h * K + i] : 1.f;
    }
    // zero the padding of both buffers once (cp.async never writes it)
    for (int i = tid; i < 2 * buf_floats; i += nthreads) smem[i] = 0.f;
    __syncthreads();

    pdl_wait();
    float S[CPT][KT];
#pragma unroll
    for (int j = 0; j < CPT; j++)
#pragma unroll
        for (int i = 0; i < KT; i++) S[j][i] = (live[j] && part * KT + i < K) ? srow[(size_t)j * K + i] : 0.f;

    // 16-byte copies where every row piece is aligned (the usual case: K, V and the row strides multiples of 4)
    const bool wide = (K % 4 == 0) && (V % 4 == 0) && (vt % 4 == 0) && (ldq % 4 == 0) && (MODE == GATE_SCALAR || ldg % 4 == 0) &&
                      (ldv % 4 == 0) && (!(MODE == GATE_EXP_EXP || READY) || ldk % 4 == 0) &&
                      ((((size_t)q | (size_t)(MODE == GATE_SCALAR ? q : g) | (size_t)v |
                         (size_t)((MODE == GATE_EXP_EXP || READY) ? k : q)) & 15) == 0);
    float bonus_r[KT];
#pragma unroll
    for (int i = 0; i < KT; i++) bonus_r[i] = c_bonus[part * KT + i];
    auto stage = [&](int buffer, int r0) {
        float* base = smem + buffer * buf_floats;
        const int count = min(CHUNK, row1 - r0);
        if (wide) {
            const int k4 = K / 4, v4 = vt / 4;
            for (int i = tid; i < count * k4; i += nthreads) {
                const int t = i / k4, c = (i - t * k4) * 4;
                const size_t r = (size_t)(r0 + t);
                cp_async16(base + t * kp + at(c), q + r * ldq + h * K + c);
                if (MODE == GATE_EXP_EXP || READY) cp_async16(base + (CHUNK + t) * kp + at(c), k + r * ldk + h * K + c);
                if (MODE != GATE_SCALAR) cp_async16(base + (2 * CHUNK + t) * kp + at(c), g + r * ldg + h * K + c);
            }
            for (int i = tid; i < count * v4; i += nthreads) {
                const int t = i / v4, c = (i - t * v4) * 4;
                if (v0 + c < V) cp_async16(base + 3 * CHUNK * kp + t * vt + c, v + (size_t)(r0 + t) * ldv + h * V + v0 + c);
            }
        } else {
            for (int i = tid; i < count * K; i += nthreads) {
                const int t = i / K, c = i - t * K;
                const size_t r = (size_t)(r0 + t);
                cp_async4(base + t * kp + at(c), q + r * ldq + h * K + c);
                if (MODE == GATE_EXP_EXP || READY) cp_async4(base + (CHUNK + t) * kp + at(c), k + r * ldk + h * K + c);
                if (MODE != GATE_SCALAR) cp_async4(base + (2 * CHUNK + t) * kp + at(c), g + r * ldg + h * K + c);
            }
            for (int i = tid; i < count * vt; i += nthreads) {
                const int t = i / vt, c = i - t * vt;
                if (v0 + c < V) cp_async4(base + 3 * CHUNK * kp + t * vt + c, v + (size_t)(r0 + t) * ldv + h * V + v0 + c);
            }
        }
        if (MODE == GATE_SCALAR && tid < count)          // the token's one decay, at the head of its row of d
            cp_async4(base + (2 * CHUNK + tid) * kp, g + (size_t)(r0 + tid) * ldg + h);
        cp_async_commit();
    };

    stage(0, row0);
    int buffer = 0;
    for (int r0 = row0; r0 < row1; r0 += CHUNK, buffer ^= 1) {
        const int count = min(CHUNK, row1 - r0);
        cp_async_wait_all();
        __syncthreads();                            // the chunk has landed; everyone is done with the other buffer
        if (r0 + CHUNK < row1) stage(buffer ^ 1, r0 + CHUNK);
        float* base = smem + buffer * buf_floats;
        float* sq = base, *sk = base + CHUNK * kp, *sd = base + 2 * CHUNK * kp, *sv = base + 3 * CHUNK * kp;
        if (!READY) {
            // gates, in place
            for (int i = tid; i < count * K; i += nthreads) {
                const int t = i / K, c = i - t * K, p = t * kp + at(c);
                const float raw = __fadd_rn(sd[p], c_bias[c]);
                if (MODE == GATE_EXP_EXP) {
                    sd[p] = gate_decay(raw);
                } else {
                    const float d = gate_lower(raw, c_lower[c]);
                    sd[p] = d;
                    sk[p] = __fsub_rn(1.0f, d);
                    sq[p] = gate_silu(sq[p]);
                }
            }
            __syncthreads();
        }
#pragma unroll SCAN_UNROLL
        for (int t = 0; t < count; t++) {
            const float4* tq = reinterpret_cast<const float4*>(sq + t * kp + part * KTP);
            const float4* tk = reinterpret_cast<const float4*>(sk + t * kp + part * KTP);
            const float4* td = reinterpret_cast<const float4*>(sd + t * kp + part * KTP);
            float vv[CPT], oe[CPT][4];
            const float d_all = MODE == GATE_SCALAR ? sd[t * kp] : 0.f;
#pragma unroll
            for (int j = 0; j < CPT; j++) {
                vv[j] = live[j] ? sv[t * vt + col + j] : 0.f;
                oe[j][0] = oe[j][1] = oe[j][2] = oe[j][3] = 0.f;
            }
#pragma unroll
            for (int i4 = 0; i4 < KT / 4; i4++) {
                const float4 q4 = tq[i4], k4 = tk[i4], d4 = MODE == GATE_SCALAR ? make_float4(d_all, d_all, d_all, d_all) : td[i4];
                const float qe[4] = {q4.x, q4.y, q4.z, q4.w}, ke[4] = {k4.x, k4.y, k4.z, k4.w}, de[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = 4 * i4 + e;
#pragma unroll
                    for (int j = 0; j < CPT; j++) {
                        const float a = ke[e] * vv[j];
                        if (MODE == GATE_EXP_EXP) {
                            oe[j][e] = fmaf(qe[e], fmaf(bonus_r[i], a, S[j][i]), oe[j][e]);
                            S[j][i] = fmaf(de[e], S[j][i], a);
                        } else {
                            S[j][i] = fmaf(de[e], S[j][i], a);
                            oe[j][e] = fmaf(qe[e], S[j][i], oe[j][e]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < CPT; j++) {
                float o = (oe[j][0] + oe[j][1]) + (oe[j][2] + oe[j][3]);
                for (int off = 1; off < ks; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
                if (live[j] && part == 0) out[(size_t)(r0 + t) * H * V + h * V + vcol + j] = o;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CPT; j++) {
        if (!live[j]) continue;
#pragma unroll
        for (int i = 0; i < KT; i++)
            if (part * KT + i < K) srow[(size_t)j * K + i] = S[j][i];
    }
}

// The gates of many rows ahead of the recurrence (the recurrence itself is a chain over the tokens; this is not).
// MODE 0: d = exp(-exp(g + bias)).  MODE 1: d = lower + (1 - lower) sigmoid(g + bias), k = 1 - d, q = silu(q).
template <int MODE>
__global__ void gate_prepare_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ g, long long ldg,
                                    const float* __restrict__ gate_bias, const float* __restrict__ lower,
                                    float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ d_out,
                                    long long rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * width;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / width;
        const int c = (int)(idx - r * width);
        const float raw = __fadd_rn(g[r * ldg + c], gate_bias ? gate_bias[c] : 0.f);
        if (MODE == GATE_EXP_EXP) {
            d_out[idx] = gate_decay(raw);
        } else {
            const float d = gate_lower(raw, lower ? lower[c] : 0.f);
            d_out[idx] = d;
            k_out[idx] = __fsub_rn(1.0f, d);
            q_out[idx] = gate_silu(q[r * ldq + c]);
        }
    }
}

// ---------------------------------------------------------------------------------------------- norm of the heads
// y[n, h, :] = o[n, h, :] / sqrt(mean(o[n, h, :]^2) + eps) * w[h * w_head_stride + :] (* silu(gate[n, h, :]), or, with
// gate_sigmoid, * sigmoid(gate[n, h, :]))
// One warp per (row, head).
template <typename T>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_head_stride,
                                         const float* __restrict__ gate, long long ldgate, T* __restrict__ y, int n_rows,
                                         int H, int V, float eps, int gate_sigmoid) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * H) return;
    const int n = warp / H, h = warp - n * H;
    const float* src = o + ((size_t)n * H + h) * V;
    float ss = 0.f;
    if (V <= 256) {
        // the head's values stay in registers: all loads in flight at once, one pass over memory
        float val[8], gz[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = lane + 32 * j;
            val[j] = i < V ? src[i] : 0.f;
            gz[j] = (gate && i < V) ? gate[(size_t)n * ldgate + h * V + i] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) ss = fmaf(val[j], val[j], ss);      // lane-wise in index order, as the loop below
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)V + eps);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = lane + 32 * j;
            if (i >= V) break;
            float r = val[j] * inv * w[h * w_head_stride + i];
            if (gate) r *= (gate_sigmoid ? 1.0f : gz[j]) / (1.0f + expf(-gz[j]));
            y[((size_t)n * H + h) * V + i] = from_f32<T>(r);
        }
        return;
    }
    for (int i = lane; i < V; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
        float r = src[i] * inv * w[h * w_head_stride + i];
        if (gate) {
            const float z = gate[(size_t)n * ldgate + h * V + i];
            r *= (gate_sigmoid ? 1.0f : z) / (1.0f + expf(-z));
        }
        y[((size_t)n * H + h) * V + i] = from_f32<T>(r);
    }
}

// ---------------------------------------------------------------------------------------------- matrix memory
// The gates of a matrix memory with exponential gating, ahead of esp_gated_scan(mode 1, ready): per head and token
//     i = cap tanh((raw_i + b_i) / cap),  f = logsigmoid(cap tanh((raw_f + b_f) / cap)),
//     m_t = max(f + m_(t-1), i),  keep = exp(f + m_(t-1) - m_t),  take = exp(i - m_t)
// First kernel: a block owns (sequence, head); the gates of 128 tokens are made in parallel, one thread then walks the
// chain of maxima (an add and a max per token, in token order, so cutting a sequence into steps changes no bit), and
// keep, take and m go out as [rows, H].  m_(t-1) of a run's first token is the sequence's state (m_state[slot *
// state_stride + h], zero in a fresh slot), which the run's last m_t replaces.
// Second kernel, over all rows at once: the values the recurrence reads, v_out = take * [v, 1, 0 ...] (V1 >= V + 1
// columns a head: the input weight rides on the values, so that the keys go in as projected; column V accumulates the
// normaliser n_t = keep n_(t-1) + take k_t as one more value column of the same recurrence; further columns are zero
// and only align the rows).  The recurrence takes keep as its one decay per head and token (mode 2).
constexpr int MM_CHUNK = 128;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

__global__ void __launch_bounds__(MM_CHUNK)
matrix_memory_gates_kernel(const float* __restrict__ gi, const float* __restrict__ gf, long long ld,
                           const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                           float* __restrict__ m_state, long long state_stride, const int* __restrict__ seq_start,
                           const int* __restrict__ seq_slot, float* __restrict__ keep_out, float* __restrict__ take_out,
                           float* __restrict__ m_out, int H) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_i[MM_CHUNK], s_f[MM_CHUNK], s_carried[MM_CHUNK], s_new[MM_CHUNK];
    __shared__ float s_m;
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = seq_start[b], row1 = seq_start[b + 1];
    if (row1 <= row0) return;
    float* mp = m_state + (size_t)seq_slot[b] * state_stride + h;
    if (tid == 0) s_m = *mp;
    const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
    for (int r0 = row0; r0 < row1; r0 += MM_CHUNK) {
        const int count = min(MM_CHUNK, row1 - r0);
        __syncthreads();
        if (tid < count) {
            const size_t r = (size_t)(r0 + tid);
            s_i[tid] = cap * tanhf((gi[r * ld + h] + bi) / cap);
            s_f[tid] = log_sigmoid(cap * tanhf((gf[r * ld + h] + bf) / cap));
        }
        __syncthreads();
        if (tid == 0) {
            float m = s_m;
#pragma unroll 8
            for (int t = 0; t < count; t++) {
                const float carried = __fadd_rn(s_f[t], m);
                m = fmaxf(carried, s_i[t]);
                s_carried[t] = carried;
                s_new[t] = m;
            }
            s_m = m;
        }
        __syncthreads();
        if (tid < count) {
            const size_t o = (size_t)(r0 + tid) * H + h;
            const float m_new = s_new[tid];
            m_out[o] = m_new;
            keep_out[o] = expf(s_carried[tid] - m_new);
            take_out[o] = expf(s_i[tid] - m_new);
        }
    }
    __syncthreads();
    if (tid == 0) *mp = s_m;
}

__global__ void matrix_memory_expand_kernel(const float* __restrict__ v, long long ld, const float* __restrict__ take,
                                            float* __restrict__ v_out, int H, int V, int V1) {
    pdl_trigger();
    pdl_wait();
    const size_t r = blockIdx.x;
    const int vw = H * V1;
    for (int c = threadIdx.x; c < vw; c += blockDim.x) {
        const int h = c / V1, j = c - h * V1;
        const float w = take[r * H + h];
        v_out[r * vw + c] = j < V ? v[r * ld + h * V + j] * w : (j == V ? w : 0.f);
    }
}

// What follows the recurrence (o has V1 columns a head; the queries went in unscaled, so o is multiplied by q_scale
// first): o[n, h, :V] / (max(|o[n, h, V]|, exp(-m[n, h])) + floor_eps), each head scaled to unit
// root mean square (eps inside the root), times a weight per channel, times sigmoid(gate).  One warp per (row, head).
template <typename T>
__global__ void matrix_memory_finish_kernel(const float* __restrict__ o, const float* __restrict__ m,
                                            const float* __restrict__ w, const float* __restrict__ gate, long long ldgate,
                                            T* __restrict__ y, int n_rows, int H, int V, int V1, float eps,
                                            float floor_eps, float q_scale) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * H) return;
    const int n = warp / H, h = warp - n * H;
    const float* src = o + ((size_t)n * H + h) * V1;
    const float den = (fmaxf(fabsf(src[V] * q_scale), expf(-m[(size_t)n * H + h])) + floor_eps) / q_scale;
    float ss = 0.f;
    if (V <= 512) {
        // the head's values stay in registers: all loads in flight at once, one pass over memory
        float val[16], gz[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int i = lane + 32 * j;
            val[j] = i < V ? src[i] / den : 0.f;
            gz[j] = (gate && i < V) ? gate[(size_t)n * ldgate + h * V + i] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; j++) ss = fmaf(val[j], val[j], ss);      // lane-wise in index order, as the loop below
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)V + eps);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int i = lane + 32 * j;
            if (i >= V) break;
            float r = val[j] * inv * w[h * V + i];
            if (gate) r *= 1.0f / (1.0f + expf(-gz[j]));
            y[((size_t)n * H + h) * V + i] = from_f32<T>(r);
        }
        return;
    }
    for (int i = lane; i < V; i += 32) {
        const float val = src[i] / den;
        ss = fmaf(val, val, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
        float r = src[i] / den * inv * w[h * V + i];
        if (gate) r *= 1.0f / (1.0f + expf(-gate[(size_t)n * ldgate + h * V + i]));
        y[((size_t)n * H + h) * V + i] = from_f32<T>(r);
    }
}

// ---------------------------------------------------------------------------------------------- gated diagonal recurrence
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The two branches ahead of the recurrence.  proj: [rows, 2C] float, the gate branch's projection in columns [0, C),
// the input branch's in [C, 2C).  gate_out = gelu_tanh(proj_y + bias_y);  u = conv_b + sum_j conv_w[c, j] * xin[t - (taps
// - 1) + j, c] with xin = proj_x + bias_x, the last column being the token's own; inputs ahead of a run's first token
// come from the sequence's state (conv_state[slot]: [taps - 1, C], oldest first; zeros in a fresh slot).  u goes out in
// 32-bit (the recurrence reads it) and in the activation dtype (the gates' projections read it).
template <typename T>
__global__ void conv_branches_kernel(const float* __restrict__ proj, const float* __restrict__ bias_y,
                                     const float* __restrict__ bias_x, const float* __restrict__ conv_w,
                                     const float* __restrict__ conv_b, const float* __restrict__ conv_state,
                                     long long state_stride, const int* __restrict__ tok_seq,
                                     const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                     float* __restrict__ gate_out, float* __restrict__ u32, T* __restrict__ u_act, int C,
                                     int taps) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n];
    const int in_run = n - seq_start[seq];
    const float* st = conv_state + (size_t)seq_slot[seq] * state_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        gate_out[(size_t)n * C + c] = gelu_tanh_f(proj[(size_t)n * 2 * C + c] + (bias_y ? bias_y[c] : 0.f));
        float u = conv_b ? conv_b[c] : 0.f;
        const float bx = bias_x ? bias_x[c] : 0.f;
        for (int j = 0; j < taps; j++) {
            const int back = taps - 1 - j;
            float xin;
            if (in_run - back >= 0) xin = proj[(size_t)(n - back) * 2 * C + C + c] + bx;
            else xin = st[(size_t)(taps - 1 + in_run - back) * C + c];
            u = fmaf(conv_w[(size_t)c * taps + j], xin, u);
        }
        u32[(size_t)n * C + c] = u;
        u_act[(size_t)n * C + c] = from_f32<T>(u);
    }
}

// conv_state[slot] <- the last taps - 1 inputs of the sequence after this step (a thread owns a channel: it reads what
// it needs of the old state before it writes).
constexpr int CONV_MAX_TAPS = 16;
__global__ void conv_state_keep_kernel(const float* __restrict__ proj, const float* __restrict__ bias_x,
                                       float* __restrict__ conv_state, long long state_stride,
                                       const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int row0 = seq_start[b], run = seq_start[b + 1] - row0;
    if (run <= 0) return;
    float* st = conv_state + (size_t)seq_slot[b] * state_stride;
    const int keep = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float next[CONV_MAX_TAPS];
        for (int j = 0; j < keep; j++) {
            const int e = run + j;                   // index in (old state, then the run's inputs)
            next[j] = e < keep ? st[(size_t)e * C + c]
                               : proj[(size_t)(row0 + e - keep) * 2 * C + C + c] + (bias_x ? bias_x[c] : 0.f);
        }
        for (int j = 0; j < keep; j++) st[(size_t)j * C + c] = next[j];
    }
}

// S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-decay_scale r_t softplus(lam)), r_t = sigmoid(raw_r + b_r),
// i_t = sigmoid(raw_i + b_i); out = S_t * gate.  gates: [rows, blocks, 2, C / blocks] float (a block's r then its i, as the
// block-diagonal projection leaves them).  Two kernels.  The first, over all rows at once, turns the raw gates into the
// recurrence's two coefficients in place: a_t where r was, sqrt(1 - a_t^2) i_t u_t where i was (1 - a^2 is taken as
// -expm1(2 ln a)).  The second is the chain itself: a thread owns (sequence, channel) and walks the run's tokens in
// order, one multiply-add a token.  A block owns 32 channels of a sequence: all its warps stage the coefficients of
// DIAG_TILE tokens at a time into one of two shared-memory buffers by cp.async, the next tile while the first warp
// walks the chain over this one, so the chain never waits for global memory.  S lives in state[slot * state_stride
// + c], 32-bit.
constexpr int DIAG_TILE = 64, DIAG_THREADS = 128;

__global__ void diag_coefficients_kernel(float* __restrict__ gates, const float* __restrict__ bias_r,
                                         const float* __restrict__ bias_i, const float* __restrict__ lam, float decay_scale,
                                         const float* __restrict__ u, int C, int cb) {
    pdl_trigger();
    pdl_wait();
    const size_t r = blockIdx.x;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const int blk = c / cb, j = c - blk * cb;
        float* g = gates + r * 2 * C + (size_t)blk * 2 * cb + j;
        const float l = lam[c];
        const float rate = decay_scale * (l > 20.f ? l : log1pf(expf(l)));
        const float rr = 1.0f / (1.0f + expf(-(g[0] + (bias_r ? bias_r[c] : 0.f))));
        const float ii = 1.0f / (1.0f + expf(-(g[cb] + (bias_i ? bias_i[c] : 0.f))));
        const float log_a = -rate * rr;
        g[0] = expf(log_a);
        g[cb] = sqrtf(-expm1f(2.0f * log_a)) * (ii * u[r * C + c]);
    }
}

template <typename T>
__global__ void __launch_bounds__(DIAG_THREADS)
diag_scan_kernel(const float* __restrict__ coef, const float* __restrict__ gate, float* __restrict__ state,
                 long long state_stride, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                 T* __restrict__ out, int C, int cb) {
    pdl_trigger();
    __shared__ float buf[2][3][DIAG_TILE][32];          // a_t, the input term, the gate branch: two tiles of tokens
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
    const int c = blockIdx.y * 32 + lane;
    const bool live = c < C;
    const int row0 = seq_start[b], row1 = seq_start[b + 1];
    if (row1 <= row0) return;
    const int blk = live ? c / cb : 0, j = live ? c - blk * cb : 0;
    const size_t goff = (size_t)blk * 2 * cb + j;
    pdl_wait();
    auto stage = [&](int which, int r0) {
        const int count = min(DIAG_TILE, row1 - r0);
        if (live) {
            for (int t = tid >> 5; t < count; t += DIAG_THREADS / 32) {
                const float* g = coef + (size_t)(r0 + t) * 2 * C + goff;
                cp_async4(&buf[which][0][t][lane], g);
                cp_async4(&buf[which][1][t][lane], g + cb);
                cp_async4(&buf[which][2][t][lane], gate + (size_t)(r0 + t) * C + c);
            }
        }
        cp_async_commit();
    };
    float* sp = state + (size_t)seq_slot[b] * state_stride + c;
    float S = (live && tid < 32) ? *sp : 0.f;
    stage(0, row0);
    int which = 0;
    for (int r0 = row0; r0 < row1; r0 += DIAG_TILE, which ^= 1) {
        const int count = min(DIAG_TILE, row1 - r0);
        cp_async_wait_all();
        __syncthreads();                                 // the tile has landed; the chain is done with the other one
        if (r0 + DIAG_TILE < row1) stage(which ^ 1, r0 + DIAG_TILE);
        if (tid < 32 && live) {
#pragma unroll 8
            for (int t = 0; t < count; t++) {
                S = fmaf(buf[which][0][t][lane], S, buf[which][1][t][lane]);
                out[(size_t)(r0 + t) * C + c] = from_f32<T>(S * buf[which][2][t][lane]);
            }
        }
    }
    if (tid < 32 && live) *sp = S;
}
}  // namespace

ESP_API int esp_token_shift_mix(const void* h, int is_bf16, const float* prev_state, long long state_stride,
                                const int* tok_seq, const int* seq_start, const int* seq_slot, const float* mu, void* out,
                                int n_mix, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, token_shift_mix_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)h,
                       prev_state, state_stride, tok_seq, seq_start, seq_slot, mu, (bf16*)out, n_mix, n_rows, width);
    else
        esp_launch_pdl(ESP_PDL_SMALL, token_shift_mix_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)h,
                       prev_state, state_stride, tok_seq, seq_start, seq_slot, mu, (float*)out, n_mix, n_rows, width);
    return esp_launch_status();
}

ESP_API int esp_token_shift_keep(const void* h, int is_bf16, float* prev_state, long long state_stride, const int* seq_start,
                                 const int* seq_slot, int n_seqs, int width, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, token_shift_keep_kernel<bf16>, dim3(n_seqs), dim3(128), 0, stream, (const bf16*)h,
                       prev_state, state_stride, seq_start, seq_slot, width);
    else
        esp_launch_pdl(ESP_PDL_SMALL, token_shift_keep_kernel<float>, dim3(n_seqs), dim3(128), 0, stream, (const float*)h,
                       prev_state, state_stride, seq_start, seq_slot, width);
    return esp_launch_status();
}

// Makes the gates of ``rows`` rows ahead of esp_gated_scan(..., ready = 1): d_out (and, mode 1, q_out and k_out), each
// float [rows, width] with width = heads * key channels.
ESP_API int esp_gate_prepare(int mode, const float* q, long long ldq, const float* g, long long ldg, const float* gate_bias,
                             const float* lower, float* q_out, float* k_out, float* d_out, long long rows, int width,
                             cudaStream_t stream) {
    if (rows <= 0) return 0;
    long long blocks = (rows * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (mode == GATE_EXP_EXP)
        esp_launch_pdl(ESP_PDL_SMALL, gate_prepare_kernel<GATE_EXP_EXP>, dim3((int)blocks), dim3(256), 0, stream, q, ldq, g, ldg,
                       gate_bias, lower, q_out, k_out, d_out, rows, width);
    else if (mode == GATE_LOWER_SIGMOID && q && q_out && k_out)
        esp_launch_pdl(ESP_PDL_SMALL, gate_prepare_kernel<GATE_LOWER_SIGMOID>, dim3((int)blocks), dim3(256), 0, stream, q, ldq, g,
                       ldg, gate_bias, lower, q_out, k_out, d_out, rows, width);
    else
        return (int)cudaErrorInvalidValue;
    return esp_launch_status();
}

// mode: 0 = decay exp(-exp(.)) with an extra weight on the token being read, 1 = lower-bounded sigmoid gate that also writes,
// 2 (with ready) = one ready-made decay per head and token, g being [rows, H]; q and k as given, the output reads S_t.
// ready: q, k and g already hold the query, the written key and the decay (esp_gate_prepare made them).
ESP_API int esp_gated_scan(int mode, int ready, const float* q, long long ldq, const float* k, long long ldk, const float* g,
                           long long ldg, const float* v, long long ldv, const float* gate_bias, const float* lower,
                           const float* bonus, float* state, long long state_stride, const int* seq_start,
                           const int* seq_slot, float* out, int n_seqs, int H, int K, int V, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (K <= 0 || V <= 0 || K > MAX_K || H > 65535) return (int)cudaErrorInvalidValue;
    int ks = 1;
    while (ks * KT < K) ks <<= 1;                  // 1, 2, 4, 8 or 16 slices of KT channels
    if (ks > 16) return (int)cudaErrorInvalidValue;
    // value columns of a block (ESP_SCAN_SMALL_THREADS < 128: smaller blocks for grids that leave SMs empty)
    int threads = SCAN_THREADS;
    if ((long long)n_seqs * H * ((V + (threads / ks) * CPT - 1) / ((threads / ks) * CPT)) < 148 && ks <= 32 && V > (64 / ks) * CPT) threads = ESP_SCAN_SMALL_THREADS;
    const int vt = (threads / ks) * CPT;
    const int vtiles = (V + vt - 1) / vt;
    const size_t smem = 2 * (size_t)CHUNK * (3 * ks * KTP + vt) * sizeof(float);
    dim3 grid(n_seqs, H, vtiles);
    if ((mode == GATE_EXP_EXP || ready) && !k) return (int)cudaErrorInvalidValue;
#define ESP_SCAN(MODE_, READY_)                                                                                              \
    {                                                                                                                       \
        auto kernel = gated_scan_kernel<MODE_, READY_>;                                                                     \
        static bool set = false;                                                                                            \
        if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); set = true; }     \
        /* a step of many rows runs long and holds its shared memory: no early start beside its predecessor */             \
        esp_launch_pdl(READY_ ? 0 : ESP_PDL_SMALL, kernel, grid, dim3(threads), smem, stream, q, ldq, k, ldk, g, ldg, v, ldv, \
                       gate_bias, lower, bonus, state, state_stride, seq_start, seq_slot, out, H, K, V, ks, vt);            \
    }
    if (mode == GATE_SCALAR && ready) ESP_SCAN(GATE_SCALAR, true)
    else if (mode == GATE_EXP_EXP && !ready) ESP_SCAN(GATE_EXP_EXP, false)
    else if (mode == GATE_EXP_EXP) ESP_SCAN(GATE_EXP_EXP, true)
    else if (mode == GATE_LOWER_SIGMOID && !ready) ESP_SCAN(GATE_LOWER_SIGMOID, false)
    else if (mode == GATE_LOWER_SIGMOID) ESP_SCAN(GATE_LOWER_SIGMOID, true)
    else return (int)cudaErrorInvalidValue;
#undef ESP_SCAN
    return esp_launch_status();
}

ESP_API int esp_head_rmsnorm_gate(const float* o, const float* w, int w_head_stride, const float* gate, long long ldgate,
                                  void* y, int y_is_bf16, int n_rows, int H, int V, float eps, int gate_sigmoid,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const long long warps = (long long)n_rows * H;
    const int blocks = (int)((warps + 7) / 8);
    if (y_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, head_rmsnorm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, w, w_head_stride,
                       gate, ldgate, (bf16*)y, n_rows, H, V, eps, gate_sigmoid);
    else
        esp_launch_pdl(ESP_PDL_SMALL, head_rmsnorm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, w, w_head_stride,
                       gate, ldgate, (float*)y, n_rows, H, V, eps, gate_sigmoid);
    return esp_launch_status();
}

// keep_take_m: 3 * rows * H floats: the decay (what esp_gated_scan mode 2 takes as g), the input weight and m_t (which
// esp_matrix_memory_finish reads) of every token and head.
ESP_API int esp_matrix_memory_prepare(const float* v, const float* gi, const float* gf, long long ld, const float* bias_i,
                                      const float* bias_f, float cap, float* m_state, long long state_stride,
                                      const int* seq_start, const int* seq_slot, float* v_out, float* keep_take_m, int n_rows,
                                      int n_seqs, int H, int V, int V1, cudaStream_t stream) {
    if (n_seqs <= 0 || n_rows <= 0) return 0;
    if (H <= 0 || H > 65535 || V <= 0 || V1 <= V || !(cap > 0.f)) return (int)cudaErrorInvalidValue;
    float* keep = keep_take_m;
    float* take = keep + (size_t)n_rows * H;
    float* m_out = take + (size_t)n_rows * H;
    esp_launch_pdl(ESP_PDL_SMALL, matrix_memory_gates_kernel, dim3(n_seqs, H), dim3(MM_CHUNK), 0, stream, gi, gf, ld, bias_i,
                   bias_f, cap, m_state, state_stride, seq_start, seq_slot, keep, take, m_out, H);
    esp_launch_pdl(ESP_PDL_SMALL, matrix_memory_expand_kernel, dim3(n_rows), dim3(256), 0, stream, v, ld, (const float*)take,
                   v_out, H, V, V1);
    return esp_launch_status();
}

ESP_API int esp_matrix_memory_finish(const float* o, const float* m, const float* w, const float* gate, long long ldgate,
                                     void* y, int y_is_bf16, int n_rows, int H, int V, int V1, float eps, float floor_eps,
                                     float q_scale, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const long long warps = (long long)n_rows * H;
    const int blocks = (int)((warps + 7) / 8);
    if (y_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, matrix_memory_finish_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, m, w, gate,
                       ldgate, (bf16*)y, n_rows, H, V, V1, eps, floor_eps, q_scale);
    else
        esp_launch_pdl(ESP_PDL_SMALL, matrix_memory_finish_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, m, w, gate,
                       ldgate, (float*)y, n_rows, H, V, V1, eps, floor_eps, q_scale);
    return esp_launch_status();
}

// Both branches of a step's rows, then the sequences' convolution states.
ESP_API int esp_conv_branches(const float* proj, const float* bias_y, const float* bias_x, const float* conv_w,
                              const float* conv_b, float* conv_state, long long state_stride, const int* tok_seq,
                              const int* seq_start, const int* seq_slot, float* gate_out, float* u32, void* u_act,
                              int act_is_bf16, int n_rows, int n_seqs, int C, int taps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || C <= 0) return (int)cudaErrorInvalidValue;
    const int threads = C >= 1024 ? 256 : 128;
    if (act_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, conv_branches_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, proj, bias_y, bias_x,
                       conv_w, conv_b, (const float*)conv_state, state_stride, tok_seq, seq_start, seq_slot, gate_out, u32,
                       (bf16*)u_act, C, taps);
    else
        esp_launch_pdl(ESP_PDL_SMALL, conv_branches_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, proj, bias_y, bias_x,
                       conv_w, conv_b, (const float*)conv_state, state_stride, tok_seq, seq_start, seq_slot, gate_out, u32,
                       (float*)u_act, C, taps);
    if (taps > 1)
        esp_launch_pdl(ESP_PDL_SMALL, conv_state_keep_kernel, dim3(n_seqs, (C + 127) / 128), dim3(128), 0, stream, proj, bias_x,
                       conv_state, state_stride, seq_start, seq_slot, C, taps);
    return esp_launch_status();
}

// gates: overwritten with the recurrence's coefficients.
ESP_API int esp_diag_scan(float* gates, const float* bias_r, const float* bias_i, const float* lam, float decay_scale,
                          const float* u, const float* gate, float* state, long long state_stride, const int* seq_start,
                          const int* seq_slot, void* out, int out_is_bf16, int n_rows, int n_seqs, int C, int blocks,
                          cudaStream_t stream) {
    if (n_seqs <= 0 || n_rows <= 0) return 0;
    if (C <= 0 || blocks <= 0 || C % blocks != 0) return (int)cudaErrorInvalidValue;
    esp_launch_pdl(ESP_PDL_SMALL, diag_coefficients_kernel, dim3(n_rows), dim3(C >= 1024 ? 256 : 128), 0, stream, gates, bias_r,
                   bias_i, lam, decay_scale, u, C, C / blocks);
    dim3 grid(n_seqs, (C + 31) / 32);
    if (out_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, diag_scan_kernel<bf16>, grid, dim3(DIAG_THREADS), 0, stream, (const float*)gates, gate, state,
                       state_stride, seq_start, seq_slot, (bf16*)out, C, C / blocks);
    else
        esp_launch_pdl(ESP_PDL_SMALL, diag_scan_kernel<float>, grid, dim3(DIAG_THREADS), 0, stream, (const float*)gates, gate, state,
                       state_stride, seq_start, seq_slot, (float*)out, C, C / blocks);
    return esp_launch_status();
}
