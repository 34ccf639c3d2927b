// The selective scan: a diagonal recurrence per (channel, state entry) whose decay and input come from the token.
//
//   dt = softplus(dt_raw)            (a step size per token and channel; dt_raw holds its bias already)
//   S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x[c] B[n]          A[c, n] = -exp(a_log[c, n])
//   y[c]    =  (sum_n S[c, n] C[n] + D[c] x[c]) * silu(z[c])
//
// Everything is 32-bit; the state belongs to the sequence (state[slot]: [C, N] floats) and every step continues from
// what the step before left there.  The recurrence is a chain over the tokens of a run: a thread keeps SLICE entries
// of one channel's state in registers for the whole run; the slices of a channel are neighbouring lanes and their
// partial sums are added by shuffles in a fixed order, so a token's result depends on nothing but the channel and
// the token.  Rows are staged CHUNK tokens at a time by cp.async into two buffers: B and C of a token once for all
// channels of the block, dt_raw, x and z for the block's channels.  What a token needs besides the state (the step
// size, dt x, silu(z)) is made for the whole chunk in a parallel pass over the staged rows; the chain itself is, per
// state entry, one exponential and two multiply-adds, four tokens' exponentials under way at once.
//
// SLICE is chosen from the state size alone (never from a step's rows), so the order of every sum is the same for
// every cutting and batching: 4 entries a thread for states up to 128 entries, which gives one sequence of a few
// thousand channels a few hundred warps, 8 up to 256 entries, 16 beyond.
#include "common.cuh"

namespace {
constexpr int SEL_THREADS = 128;
constexpr int SEL_CHUNK = 16;        // tokens staged at a time
constexpr int SEL_GROUP = 4;         // tokens whose exponentials are made together
constexpr int SEL_MAX_STATE = 512;   // 32 lanes of 16 entries

__device__ __forceinline__ void sel_cp4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void sel_cp16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void sel_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void sel_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// 2^v by the special-function unit (about two units in the last place; results below the normal range become zero, which
// is what a decay that small is)
__device__ __forceinline__ float sel_exp2(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

// 2^v for v <= 0 from multiply-adds alone, to within about one unit in the last place: v = n + f with n whole and
// |f| <= 1/2, 2^f by the series of exp(f ln 2) up to the seventh power (the next term is below 5e-9), the exponent
// added to the result's.  The special-function unit's 2^v is off by up to 2^-22.5, and by the same amount whenever the
// argument is the same: a state entry that keeps most of itself for hundreds of tokens multiplies as many such factors,
// and their errors add up instead of averaging out (the 32-bit engine's residual stream behind a scan of 1,100 tokens was
// 2.6 times as far from a 64-bit run as a plain 32-bit implementation's).  The 32-bit engine takes this form.
__device__ __forceinline__ float sel_exp2_series(float v) {
    v = fmaxf(v, -126.0f);                       // below that the result leaves the normal range: it is nothing either way
    const float n = rintf(v);
    const float f = v - n;                       // exact
    float p = 1.525273380405984e-05f;
    p = fmaf(p, f, 1.5403530393381608e-04f);
    p = fmaf(p, f, 1.3333558146428443e-03f);
    p = fmaf(p, f, 9.618129107628477e-03f);
    p = fmaf(p, f, 5.550410866482158e-02f);
    p = fmaf(p, f, 2.402265069591007e-01f);
    p = fmaf(p, f, 6.931471805599453e-01f);
    p = fmaf(p, f, 1.0f);
    return __int_as_float(__float_as_int(p) + ((int)n << 23));
}
template <typename TY> __device__ __forceinline__ float sel_decay(float v);
template <> __device__ __forceinline__ float sel_decay<float>(float v) { return sel_exp2_series(v); }
template <> __device__ __forceinline__ float sel_decay<bf16>(float v) { return sel_exp2(v); }

__device__ __forceinline__ float sel_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (channel tiles, sequences); block SEL_THREADS = cpb channels x L lanes a channel
template <typename TY, int SLICE>
__global__ void __launch_bounds__(SEL_THREADS)
selective_scan_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ dt_raw, long long lddt,
                      const float* __restrict__ bc, long long ldbc, const float* __restrict__ z, long long ldz,
                      const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
                      long long state_stride, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                      TY* __restrict__ y, int C, int N, int L, int vec_bc, int vec_ch) {
    pdl_trigger();
    extern __shared__ __align__(16) float sel_smem[];
    const int cpb = SEL_THREADS / L;
    const int tid = threadIdx.x, sub = tid % L, ch_local = tid / L;
    const int c = blockIdx.x * cpb + ch_local;
    const bool live = c < C;
    const int n0 = sub * SLICE;
    // per buffer: [CHUNK][2N] B and C, then [CHUNK][cpb] of dt (staged raw), x, silu(z) (staged z), dt x
    const int buf_floats = SEL_CHUNK * (2 * N + 4 * cpb);
    // exp(dt A) = 2^(dt A log2(e)): the decay rates are kept times log2(e)
    float A2[SLICE], S[SLICE];
#pragma unroll
    for (int j = 0; j < SLICE; j++) {
        const int n = n0 + j;
        A2[j] = (live && n < N) ? -expf(a_log[(size_t)c * N + n]) * 1.4426950408889634f : 0.f;   // weights: no kernel writes them
    }
    const float dsk = live ? d_skip[c] : 0.f;
    pdl_wait();
    const int seq = blockIdx.y;
    const int row0 = seq_start[seq], row1 = seq_start[seq + 1];
    if (row0 >= row1) return;
    float* st = state + (size_t)seq_slot[seq] * state_stride + (size_t)(live ? c : 0) * N;
#pragma unroll
    for (int j = 0; j < SLICE; j++) S[j] = (live && n0 + j < N) ? st[n0 + j] : 0.f;
    const int c_first = blockIdx.x * cpb;
    const int chans = min(cpb, C - c_first);
    const bool whole = n0 + SLICE <= N;

    auto stage = [&](int buf, int first) {
        float* base = sel_smem + buf * buf_floats;
        const int count = min(SEL_CHUNK, row1 - first);
        // 16-byte pieces where the rows allow them (the host says so from sizes and alignment alone), else word by word
        if (vec_bc) {
            const int pieces = N / 2;
            for (int i = tid; i < count * pieces; i += SEL_THREADS) {
                const int t = i / pieces, e = (i - t * pieces) * 4;
                sel_cp16(base + t * 2 * N + e, bc + (size_t)(first + t) * ldbc + e);
            }
        } else {
            for (int i = tid; i < count * 2 * N; i += SEL_THREADS) {
                const int t = i / (2 * N), e = i - t * 2 * N;
                sel_cp4(base + i, bc + (size_t)(first + t) * ldbc + e);
            }
        }
        float* per = base + SEL_CHUNK * 2 * N;
        if (vec_ch) {
            const int pieces = cpb / 4;
            for (int i = tid; i < count * pieces; i += SEL_THREADS) {
                const int t = i / pieces, e = (i - t * pieces) * 4;
                if (e >= chans) continue;
                const size_t r = (size_t)(first + t);
                sel_cp16(per + t * cpb + e, dt_raw + r * lddt + c_first + e);
                sel_cp16(per + SEL_CHUNK * cpb + t * cpb + e, x + r * ldx + c_first + e);
                sel_cp16(per + 2 * SEL_CHUNK * cpb + t * cpb + e, z + r * ldz + c_first + e);
            }
        } else {
            for (int i = tid; i < count * cpb; i += SEL_THREADS) {
                const int t = i / cpb, e = i - t * cpb;
                if (e >= chans) continue;
                const size_t r = (size_t)(first + t);
                sel_cp4(per + i, dt_raw + r * lddt + c_first + e);
                sel_cp4(per + SEL_CHUNK * cpb + i, x + r * ldx + c_first + e);
                sel_cp4(per + 2 * SEL_CHUNK * cpb + i, z + r * ldz + c_first + e);
            }
        }
        sel_commit();
    };

    stage(0, row0);
    int buf = 0;
    for (int first = row0; first < row1; first += SEL_CHUNK, buf ^= 1) {
        sel_wait_all();
        __syncthreads();                              // this chunk has landed; the other buffer's readers are done
        if (first + SEL_CHUNK < row1) stage(buf ^ 1, first + SEL_CHUNK);
        float* base = sel_smem + buf * buf_floats;
        float* per = base + SEL_CHUNK * 2 * N;
        const int count = min(SEL_CHUNK, row1 - first);
        // what the chain needs of a token and channel, made once for all lanes of the channel
        for (int i = tid; i < count * cpb; i += SEL_THREADS) {
            const int e = i % cpb;
            if (e >= chans) continue;
            const float dt = sel_softplus(per[i]);
            const float zv = per[2 * SEL_CHUNK * cpb + i];
            per[i] = dt;
            per[3 * SEL_CHUNK * cpb + i] = dt * per[SEL_CHUNK * cpb + i];
            per[2 * SEL_CHUNK * cpb + i] = zv / (1.0f + expf(-zv));
        }
        __syncthreads();
        for (int t0 = 0; t0 < count; t0 += SEL_GROUP) {
            float decay[SEL_GROUP][SLICE];
#pragma unroll
            for (int u = 0; u < SEL_GROUP; u++) {
                const float dt = t0 + u < count ? per[(t0 + u) * cpb + ch_local] : 0.f;
#pragma unroll
                for (int j = 0; j < SLICE; j++) decay[u][j] = sel_decay<TY>(dt * A2[j]);
            }
            float acc[SEL_GROUP];
#pragma unroll
            for (int u = 0; u < SEL_GROUP; u++) {
                acc[u] = 0.f;
                if (t0 + u < count) {
                    const float dx = per[3 * SEL_CHUNK * cpb + (t0 + u) * cpb + ch_local];
                    const float* Bt = base + (t0 + u) * 2 * N;
                    const float* Ct = Bt + N;
                    if (whole) {                     // every entry of this thread's slice exists: no test per entry
#pragma unroll
                        for (int j = 0; j < SLICE; j++) {
                            S[j] = fmaf(decay[u][j], S[j], dx * Bt[n0 + j]);
                            acc[u] = fmaf(S[j], Ct[n0 + j], acc[u]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < SLICE; j++) {
                            const int n = n0 + j;
                            if (n < N) {
                                S[j] = fmaf(decay[u][j], S[j], dx * Bt[n]);
                                acc[u] = fmaf(S[j], Ct[n], acc[u]);
                            }
                        }
                    }
                }
            }
            for (int o = 1; o < L; o <<= 1) {
#pragma unroll
                for (int u = 0; u < SEL_GROUP; u++) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
            }
            if (sub == 0 && live) {
#pragma unroll
                for (int u = 0; u < SEL_GROUP; u++) {
                    if (t0 + u < count) {
                        const float xv = per[SEL_CHUNK * cpb + (t0 + u) * cpb + ch_local];
                        const float gz = per[2 * SEL_CHUNK * cpb + (t0 + u) * cpb + ch_local];
                        y[(size_t)(first + t0 + u) * C + c] = from_f32<TY>(fmaf(dsk, xv, acc[u]) * gz);
                    }
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < SLICE; j++)
            if (n0 + j < N) st[n0 + j] = S[j];
    }
}

template <typename TY, int SLICE>
void selective_scan_launch(dim3 grid, size_t smem, cudaStream_t stream, const float* x, long long ldx, const float* dt_raw,
                           long long lddt, const float* bc, long long ldbc, const float* z, long long ldz, const float* a_log,
                           const float* d_skip, float* state, long long state_stride, const int* seq_start,
                           const int* seq_slot, void* y, int C, int N, int L, int vec_bc, int vec_ch) {
    static bool raised = false;        // per instantiation
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(selective_scan_kernel<TY, SLICE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    esp_launch_pdl(ESP_PDL_SMALL, selective_scan_kernel<TY, SLICE>, grid, dim3(SEL_THREADS), smem, stream, x, ldx, dt_raw, lddt,
                   bc, ldbc, z, ldz, a_log, d_skip, state, state_stride, seq_start, seq_slot, (TY*)y, C, N, L, vec_bc, vec_ch);
}
}  // namespace

// x, dt_raw, z: float rows [rows, C] with their strides; bc: float rows whose first N values are B and next N are C;
// a_log [C, N]; d_skip [C]; state rows of at least C * N floats; y [rows, C] float or bfloat16.
ESP_API int esp_selective_scan(const float* x, long long ldx, const float* dt_raw, long long lddt, const float* bc,
                               long long ldbc, const float* z, long long ldz, const float* a_log, const float* d_skip,
                               float* state, long long state_stride, const int* seq_start, const int* seq_slot, void* y,
                               int y_is_bf16, int n_seqs, int C, int N, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (C <= 0 || N <= 0 || N > SEL_MAX_STATE || n_seqs > 65535) return (int)cudaErrorInvalidValue;
    const int slice = N <= 128 ? 4 : N <= 256 ? 8 : 16;      // from the state size alone: see the top
    int L = 1;
    while (L * slice < N) L <<= 1;
    const int cpb = SEL_THREADS / L;
    const size_t smem = (size_t)2 * SEL_CHUNK * (2 * N + 4 * cpb) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid((C + cpb - 1) / cpb, n_seqs);
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec_bc = (N % 2 == 0 && ldbc % 4 == 0 && aligned(bc)) ? 1 : 0;
    const int vec_ch = (C % 4 == 0 && cpb % 4 == 0 && ldx % 4 == 0 && lddt % 4 == 0 && ldz % 4 == 0 && aligned(x) && aligned(dt_raw) &&
                        aligned(z)) ? 1 : 0;
#define ESP_SEL(TY, SLICE)                                                                                                   \
    selective_scan_launch<TY, SLICE>(grid, smem, stream, x, ldx, dt_raw, lddt, bc, ldbc, z, ldz, a_log, d_skip, state,        \
                                     state_stride, seq_start, seq_slot, y, C, N, L, vec_bc, vec_ch)
    if (y_is_bf16) {
        if (slice == 4) ESP_SEL(bf16, 4);
        else if (slice == 8) ESP_SEL(bf16, 8);
        else ESP_SEL(bf16, 16);
    } else {
        if (slice == 4) ESP_SEL(float, 4);
        else if (slice == 8) ESP_SEL(float, 8);
        else ESP_SEL(float, 16);
    }
#undef ESP_SEL
    return esp_launch_status();
}
