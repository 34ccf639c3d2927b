// The delta rule with a decay per key channel, and what stands around it: a short causal convolution with an
// activation, the unit vectors and gates it reads, and the decay of gated linear attention.
//
//     S <- diag(d_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S: [K, V] per head
//
// Everything that enters the recurrence is 32-bit and the recurrence is a chain over the tokens, so it runs on the
// CUDA cores in the same arrangement as the gated outer-product recurrence of recurrent.cu: a block owns (sequence,
// value head, a tile of value columns), a thread one value column and a slice of KT key channels that it keeps in
// registers for the whole run of tokens; the slices of a column are neighbouring lanes.  A token costs two sums over
// the key channels (S^T k before the write, S^T q after it), each added over the slices by shuffles whose result
// every lane of the column receives.  Rows are staged CHUNK tokens at a time by cp.async into two buffers.  The order
// of every addition depends on the token and the channel alone: cutting a sequence into steps, or batching it with
// others, changes no bit.  Several value heads may read one query/key head.
#include "common.cuh"

namespace {

constexpr int DELTA_THREADS = 128;
constexpr int KT = 16;          // key channels a thread keeps
constexpr int KTP = KT + 4;     // a slice's stride in shared memory: slices 80 bytes apart fall into different banks
constexpr int CHUNK = 16;       // tokens staged at a time
constexpr int MAX_K = 16 * KT;  // key channels of a head that the kernel takes

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

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// q, k: [rows, ld*] float, G heads of K channels (value head h reads head h / (H / G)); d: [rows, ldd], H heads of K;
// v: [rows, ldv], H heads of V; beta: [rows, H].  state: [slots, state_stride] floats, the head's block at h*V*K laid
// out [V][K] (a thread's key slice is contiguous).  out: [rows, H*V] float.
__global__ void __launch_bounds__(DELTA_THREADS)
delta_scan_kernel(const float* __restrict__ q, long long ldq, const float* __restrict__ k, long long ldk,
                  const float* __restrict__ d, long long ldd, const float* __restrict__ v, long long ldv,
                  const float* __restrict__ beta, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ out, int H, int G,
                  int K, int V, int ks, int vt) {
    pdl_trigger();
    extern __shared__ __align__(16) float smem[];
    const int kp = ks * KTP;                       // floats of one token's q (or k, or d): the threads' slices, padded
    auto at = [](int c) { return (c / KT) * KTP + (c % KT); };     // where key channel c lies in such a row
    // per buffer: q[CHUNK][kp], k[CHUNK][kp], d[CHUNK][kp], v[CHUNK][vt], beta[CHUNK]
    const int buf_floats = CHUNK * (3 * kp + vt + 1);
    const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * vt;
    const int g = h / (H / G);
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int part = tid % ks, col = tid / ks;     // neighbouring lanes hold the slices of one column
    const int vcol = v0 + col;
    const bool live = col < vt && vcol < V;
    const int row0 = seq_start[b], row1 = seq_start[b + 1];
    if (row1 <= row0) return;
    float* srow = state + (size_t)seq_slot[b] * state_stride + ((size_t)h * V + (live ? vcol : 0)) * K + part * KT;
    for (int i = tid; i < 2 * buf_floats; i += nthreads) smem[i] = 0.f;      // the padding is never written by cp.async
    __syncthreads();

    pdl_wait();
    float S[KT];
#pragma unroll
    for (int i = 0; i < KT; i++) S[i] = (live && part * KT + i < K) ? srow[i] : 0.f;

    const bool wide = (K % 4 == 0) && (V % 4 == 0) && (vt % 4 == 0) && (ldq % 4 == 0) && (ldk % 4 == 0) && (ldd % 4 == 0) &&
                      (ldv % 4 == 0) && ((((size_t)q | (size_t)k | (size_t)d | (size_t)v) & 15) == 0);
    auto stage = [&](int buffer, int r0) {
        float* base = smem + buffer * buf_floats;
        const int count = min(CHUNK, row1 - r0);
        if (wide) {
            const int k4 = K / 4, v4 = vt / 4;
            for (int i = tid; i < count * k4; i += nthreads) {
                const int t = i / k4, c = (i - t * k4) * 4;
                const size_t r = (size_t)(r0 + t);
                cp_async16(base + t * kp + at(c), q + r * ldq + g * K + c);
                cp_async16(base + (CHUNK + t) * kp + at(c), k + r * ldk + g * K + c);
                cp_async16(base + (2 * CHUNK + t) * kp + at(c), d + r * ldd + h * K + c);
            }
            for (int i = tid; i < count * v4; i += nthreads) {
                const int t = i / v4, c = (i - t * v4) * 4;
                if (v0 + c < V) cp_async16(base + 3 * CHUNK * kp + t * vt + c, v + (size_t)(r0 + t) * ldv + h * V + v0 + c);
            }
        } else {
            for (int i = tid; i < count * K; i += nthreads) {
                const int t = i / K, c = i - t * K;
                const size_t r = (size_t)(r0 + t);
                cp_async4(base + t * kp + at(c), q + r * ldq + g * K + c);
                cp_async4(base + (CHUNK + t) * kp + at(c), k + r * ldk + g * K + c);
                cp_async4(base + (2 * CHUNK + t) * kp + at(c), d + r * ldd + h * K + c);
            }
            for (int i = tid; i < count * vt; i += nthreads) {
                const int t = i / vt, c = i - t * vt;
                if (v0 + c < V) cp_async4(base + 3 * CHUNK * kp + t * vt + c, v + (size_t)(r0 + t) * ldv + h * V + v0 + c);
            }
        }
        if (tid < count) cp_async4(base + CHUNK * (3 * kp + vt) + tid, beta + (size_t)(r0 + tid) * H + h);
        cp_async_commit();
    };

    stage(0, row0);
    int buffer = 0;
    for (int r0 = row0; r0 < row1; r0 += CHUNK, buffer ^= 1) {
        const int count = min(CHUNK, row1 - r0);
        cp_async_wait_all();
        __syncthreads();                            // the chunk has landed; everyone is done with the other buffer
        if (r0 + CHUNK < row1) stage(buffer ^ 1, r0 + CHUNK);
        const float* base = smem + buffer * buf_floats;
        const float* sq = base, *sk = base + CHUNK * kp, *sd = base + 2 * CHUNK * kp, *sv = base + 3 * CHUNK * kp;
        const float* sb = base + CHUNK * (3 * kp + vt);
#pragma unroll 2
        for (int t = 0; t < count; t++) {
            const float4* tq = reinterpret_cast<const float4*>(sq + t * kp + part * KTP);
            const float4* tk = reinterpret_cast<const float4*>(sk + t * kp + part * KTP);
            const float4* td = reinterpret_cast<const float4*>(sd + t * kp + part * KTP);
            const float vv = live ? sv[t * vt + col] : 0.f;
            const float bt = sb[t];
            float ke[KT], pe[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < KT / 4; i4++) {
                const float4 k4 = tk[i4], d4 = td[i4];
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = 4 * i4 + e;
                    ke[i] = kk[e];
                    S[i] = S[i] * dd[e];
                    pe[e] = fmaf(S[i], kk[e], pe[e]);
                }
            }
            float seen = (pe[0] + pe[1]) + (pe[2] + pe[3]);                    // S^T k over this slice
            for (int off = 1; off < ks; off <<= 1) seen += __shfl_xor_sync(0xffffffffu, seen, off);
            const float u = bt * (vv - seen);
            float oe[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < KT / 4; i4++) {
                const float4 q4 = tq[i4];
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = 4 * i4 + e;
                    S[i] = fmaf(ke[i], u, S[i]);
                    oe[e] = fmaf(S[i], qq[e], oe[e]);
                }
            }
            float o = (oe[0] + oe[1]) + (oe[2] + oe[3]);
            for (int off = 1; off < ks; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (live && part == 0) out[(size_t)(r0 + t) * H * V + h * V + vcol] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < KT; i++)
            if (part * KT + i < K) srow[i] = S[i];
    }
}

// What the delta rule reads, from the rows that the convolution left (in place): q and k (G heads of K channels each,
// q at column 0 and k at column G*K of ``qk``) become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q times
// q_scale; decay[n, h, c] = exp(-exp(a_log[h]) softplus(raw[n, h, c] + dt_bias[h, c])); beta = sigmoid of
// the raw column.  One block per row, a warp per head.
__global__ void delta_prepare_kernel(float* __restrict__ qk, long long ldqk, int G, int K, float unit_eps, float q_scale,
                                     const float* __restrict__ raw, long long ldraw, float* __restrict__ decay,
                                     const float* __restrict__ dt_bias,
                                     const float* __restrict__ a_log, const float* __restrict__ b_raw, long long ldb,
                                     float* __restrict__ beta, int H) {
    pdl_trigger();
    pdl_wait();
    const size_t n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int job = warp; job < 2 * G; job += nwarp) {
        float* x = qk + n * ldqk + (size_t)job * K;
        float ss = 0.f;
        for (int i = lane; i < K; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float f = (job < G ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        for (int i = lane; i < K; i += 32) x[i] = x[i] * f;
    }
    for (int e = threadIdx.x; e < H * K; e += blockDim.x) {
        const int h = e / K;
        const float rate = expf(a_log[h]);
        decay[n * H * K + e] = expf(-rate * softplus_f(raw[n * ldraw + e] + dt_bias[e]));
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) beta[n * H + h] = sigmoid_f(b_raw[n * ldb + h]);
}

// Gated linear attention's decay and query: d = sigmoid(z + bias)^(1/tau), taken as exp(log sigmoid(.) / tau), in
// place; q_out = q * q_scale.
__global__ void channel_decay_prepare_kernel(float* __restrict__ z, const float* __restrict__ bias, float inv_tau,
                                             const float* __restrict__ q, long long ldq, float q_scale,
                                             float* __restrict__ q_out, long long rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * width;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / width;
        const int c = (int)(idx - r * width);
        z[idx] = expf(log_sigmoid_f(z[idx] + (bias ? bias[c] : 0.f)) * inv_tau);
        q_out[idx] = q[r * ldq + c] * q_scale;
    }
}

// y[n, c] = act(sum_j w[c, j] x[n - (taps - 1) + j, c]) over the rows of a sequence, the last column of w being the
// token's own; inputs ahead of a run's first token come from the sequence's state (state[slot]: [taps - 1, C],
// oldest first; zeros in a fresh slot).  bias (may be null): a number per channel added to the sum before the
// activation.  act: 0 none, 1 SiLU.  x: float rows with stride ldx; y: float [rows, C].
__global__ void causal_conv_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                                   const float* __restrict__ bias,
                                   const float* __restrict__ conv_state, long long state_stride,
                                   const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_slot, float* __restrict__ y, int C, int taps, int act) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n];
    const int in_run = n - seq_start[seq];
    const float* st = conv_state + (size_t)seq_slot[seq] * state_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float u = 0.f;
        for (int j = 0; j < taps; j++) {
            const int back = taps - 1 - j;
            const float xin = in_run - back >= 0 ? x[(size_t)(n - back) * ldx + c] : st[(size_t)(taps - 1 + in_run - back) * C + c];
            u = fmaf(w[(size_t)c * taps + j], xin, u);
        }
        if (bias) u += bias[c];
        y[(size_t)n * C + c] = act == 1 ? u * sigmoid_f(u) : u;
    }
}

// The same convolution for a reach known at compile time and rows whose pieces of four channels are aligned: a block
// takes CONV_TILE_ROWS rows and a thread four channels of them, with the last TAPS inputs of its channels in registers.
// Stepping to the next row shifts that window and loads one row; a row that opens a sequence's run (or the tile) fills
// it from the earlier rows or the sequence's state.  Per element the sum runs over the taps in the order of the kernel
// above.
constexpr int CONV_TILE_ROWS = 8;
template <int TAPS>
__global__ void __launch_bounds__(64)
causal_conv_tile_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w,
                        const float* __restrict__ bias,
                        const float* __restrict__ conv_state, long long state_stride,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_slot, float* __restrict__ y, int n_rows, int C, int act) {
    pdl_trigger();
    const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (c >= C) return;
    float wt[4][TAPS];
#pragma unroll
    for (int e = 0; e < 4; e++)
#pragma unroll
        for (int j = 0; j < TAPS; j++) wt[e][j] = w[(size_t)(c + e) * TAPS + j];
    float bs[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias) {
#pragma unroll
        for (int e = 0; e < 4; e++) bs[e] = bias[c + e];
    }
    pdl_wait();
    const int first = blockIdx.x * CONV_TILE_ROWS;
    const int last = min(first + CONV_TILE_ROWS, n_rows);
    float4 own[CONV_TILE_ROWS];                         // the tile's own inputs, all loads in flight together
#pragma unroll
    for (int i = 0; i < CONV_TILE_ROWS; i++)
        own[i] = first + i < last ? *reinterpret_cast<const float4*>(x + (size_t)(first + i) * ldx + c)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 win[TAPS];                                   // win[j]: the input `TAPS - 1 - j` rows back
#pragma unroll
    for (int i = 0; i < CONV_TILE_ROWS; i++) {
        const int n = first + i;
        if (n >= last) break;
        const int seq = tok_seq[n];
        const int in_run = n - seq_start[seq];
        if (n == first || in_run == 0) {
            const float* st = conv_state + (size_t)seq_slot[seq] * state_stride;
#pragma unroll
            for (int j = 0; j < TAPS - 1; j++) {
                const int back = TAPS - 1 - j;
                win[j] = *reinterpret_cast<const float4*>(in_run - back >= 0 ? x + (size_t)(n - back) * ldx + c
                                                                              : st + (size_t)(TAPS - 1 + in_run - back) * C + c);
            }
        }
        win[TAPS - 1] = own[i];
        float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < TAPS; j++) {
            u[0] = fmaf(wt[0][j], win[j].x, u[0]);
            u[1] = fmaf(wt[1][j], win[j].y, u[1]);
            u[2] = fmaf(wt[2][j], win[j].z, u[2]);
            u[3] = fmaf(wt[3][j], win[j].w, u[3]);
        }
        if (bias) {
#pragma unroll
            for (int e = 0; e < 4; e++) u[e] += bs[e];
        }
        if (act == 1) {
#pragma unroll
            for (int e = 0; e < 4; e++) u[e] = u[e] * sigmoid_f(u[e]);
        }
        *reinterpret_cast<float4*>(y + (size_t)n * C + c) = make_float4(u[0], u[1], u[2], u[3]);
#pragma unroll
        for (int j = 0; j < TAPS - 1; j++) win[j] = win[j + 1];
    }
}

template <int TAPS>
static void causal_conv_tile_launch(const float* x, long long ldx, const float* w, const float* bias, const float* conv_state,
                                    long long state_stride, const int* tok_seq, const int* seq_start, const int* seq_slot,
                                    float* y, int n_rows, int C, int act, cudaStream_t stream) {
    esp_launch_pdl(ESP_PDL_SMALL, causal_conv_tile_kernel<TAPS>,
                   dim3((n_rows + CONV_TILE_ROWS - 1) / CONV_TILE_ROWS, (C / 4 + 63) / 64), dim3(64), 0, stream, x, ldx, w,
                   bias, conv_state, state_stride, tok_seq, seq_start, seq_slot, y, n_rows, C, act);
}

// state[slot] <- the last taps - 1 inputs of the sequence after this step (a thread owns a channel: it reads what it
// needs of the old state before it writes).
constexpr int CONV_MAX_TAPS = 16;
__global__ void causal_conv_keep_kernel(const float* __restrict__ x, long long ldx, float* __restrict__ conv_state,
                                        long long state_stride, const int* __restrict__ seq_start,
                                        const int* __restrict__ seq_slot, int C, int taps) {
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
            next[j] = e < keep ? st[(size_t)e * C + c] : x[(size_t)(row0 + e - keep) * ldx + c];
        }
        for (int j = 0; j < keep; j++) st[(size_t)j * C + c] = next[j];
    }
}
}  // namespace

ESP_API int esp_delta_scan(const float* q, long long ldq, const float* k, long long ldk, const float* d, long long ldd,
                           const float* v, long long ldv, const float* beta, float* state, long long state_stride,
                           const int* seq_start, const int* seq_slot, float* out, int n_seqs, int H, int G, int K, int V,
                           cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (K <= 0 || V <= 0 || K > MAX_K || H > 65535 || G <= 0 || H % G != 0) return (int)cudaErrorInvalidValue;
    int ks = 1;
    while (ks * KT < K) ks <<= 1;                  // 1, 2, 4, 8 or 16 slices of KT channels
    int threads = DELTA_THREADS;
    // smaller blocks when the grid would leave SMs empty
    while (threads > 32 && threads / ks > 1 && (long long)n_seqs * H * ((V + threads / ks - 1) / (threads / ks)) < 148 &&
           V > threads / ks / 2)
        threads /= 2;
    if (threads < ks) threads = ks;
    const int vt = threads / ks;
    const int vtiles = (V + vt - 1) / vt;
    const size_t smem = 2 * (size_t)CHUNK * (3 * ks * KTP + vt + 1) * sizeof(float);
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); set = true; }
    dim3 grid(n_seqs, H, vtiles);
    esp_launch_pdl(0, delta_scan_kernel, grid, dim3(threads), smem, stream, q, ldq, k, ldk, d, ldd, v, ldv, beta, state,
                   state_stride, seq_start, seq_slot, out, H, G, K, V, ks, vt);
    return esp_launch_status();
}

ESP_API int esp_delta_prepare(float* qk, long long ldqk, int G, int K, float unit_eps, float q_scale, const float* raw,
                              long long ldraw, float* decay, const float* dt_bias, const float* a_log, const float* b_raw, long long ldb, float* beta,
                              int H, int n_rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (G <= 0 || K <= 0 || H <= 0) return (int)cudaErrorInvalidValue;
    esp_launch_pdl(ESP_PDL_SMALL, delta_prepare_kernel, dim3(n_rows), dim3(H * K >= 1024 ? 256 : 128), 0, stream, qk, ldqk, G, K,
                   unit_eps, q_scale, raw, ldraw, decay, dt_bias, a_log, b_raw, ldb, beta, H);
    return esp_launch_status();
}

ESP_API int esp_channel_decay_prepare(float* z, const float* bias, float tau, const float* q, long long ldq, float q_scale,
                                      float* q_out, long long rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!(tau > 0.f)) return (int)cudaErrorInvalidValue;
    long long blocks = (rows * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    esp_launch_pdl(ESP_PDL_SMALL, channel_decay_prepare_kernel, dim3((int)blocks), dim3(256), 0, stream, z, bias, 1.0f / tau, q, ldq,
                   q_scale, q_out, rows, width);
    return esp_launch_status();
}

// The convolution of a step's rows, then the sequences' convolution states.
ESP_API int esp_causal_conv(const float* x, long long ldx, const float* w, const float* bias, float* conv_state, long long state_stride,
                            const int* tok_seq, const int* seq_start, const int* seq_slot, float* y, int n_rows, int n_seqs,
                            int C, int taps, int act, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || C <= 0) return (int)cudaErrorInvalidValue;
    // which form runs depends on the sizes and the buffers' alignment alone, never on the rows of a step
    const bool tiled = taps >= 2 && taps <= 4 && C % 4 == 0 && ldx % 4 == 0 && state_stride % 4 == 0 &&
                       (((size_t)x | (size_t)conv_state | (size_t)y) & 15) == 0;     // bias: scalar loads
#define ESP_CONV_TILE(N)                                                                                               \
    causal_conv_tile_launch<N>(x, ldx, w, bias, (const float*)conv_state, state_stride, tok_seq, seq_start, seq_slot, y, n_rows, C, \
                               act, stream)
    if (tiled && taps == 2) ESP_CONV_TILE(2);
    else if (tiled && taps == 3) ESP_CONV_TILE(3);
    else if (tiled) ESP_CONV_TILE(4);
    else
        esp_launch_pdl(ESP_PDL_SMALL, causal_conv_kernel, dim3(n_rows), dim3(C >= 1024 ? 256 : 128), 0, stream, x, ldx, w,
                       bias, (const float*)conv_state, state_stride, tok_seq, seq_start, seq_slot, y, C, taps, act);
#undef ESP_CONV_TILE
    if (taps > 1)
        esp_launch_pdl(ESP_PDL_SMALL, causal_conv_keep_kernel, dim3(n_seqs, (C + 127) / 128), dim3(128), 0, stream, x, ldx,
                       conv_state, state_stride, seq_start, seq_slot, C, taps);
    return esp_launch_status();
}
