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
// channels of the block, dt_raw, x and z for the block's channels.
#include "common.cuh"

namespace {
constexpr int SEL_THREADS = 128;
constexpr int SEL_CHUNK = 16;        // tokens staged at a time
constexpr int SEL_SLICE = 16;        // state entries a thread keeps
constexpr int SEL_MAX_STATE = 512;   // 32 lanes of SEL_SLICE entries

__device__ __forceinline__ void sel_cp4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void sel_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void sel_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ float sel_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (channel tiles, sequences); block SEL_THREADS = cpb channels x L lanes a channel
template <typename TY>
__global__ void __launch_bounds__(SEL_THREADS)
selective_scan_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ dt_raw, long long lddt,
                      const float* __restrict__ bc, long long ldbc, const float* __restrict__ z, long long ldz,
                      const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
                      long long state_stride, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                      TY* __restrict__ y, int C, int N, int L) {
    pdl_trigger();
    extern __shared__ float sel_smem[];
    const int cpb = SEL_THREADS / L;
    const int tid = threadIdx.x, sub = tid % L, ch_local = tid / L;
    const int c = blockIdx.x * cpb + ch_local;
    const bool live = c < C;
    const int n0 = sub * SEL_SLICE;
    // per buffer: [CHUNK][2N] B and C, then [CHUNK][cpb] of dt_raw, x, z
    const int buf_floats = SEL_CHUNK * (2 * N + 3 * cpb);
    float A[SEL_SLICE], S[SEL_SLICE];
#pragma unroll
    for (int j = 0; j < SEL_SLICE; j++) {
        const int n = n0 + j;
        A[j] = (live && n < N) ? -expf(a_log[(size_t)c * N + n]) : 0.f;      // weights: no kernel writes them
    }
    const float dsk = live ? d_skip[c] : 0.f;
    pdl_wait();
    const int seq = blockIdx.y;
    const int row0 = seq_start[seq], row1 = seq_start[seq + 1];
    if (row0 >= row1) return;
    float* st = state + (size_t)seq_slot[seq] * state_stride + (size_t)(live ? c : 0) * N;
#pragma unroll
    for (int j = 0; j < SEL_SLICE; j++) S[j] = (live && n0 + j < N) ? st[n0 + j] : 0.f;

    auto stage = [&](int buf, int first) {
        float* base = sel_smem + buf * buf_floats;
        const int count = min(SEL_CHUNK, row1 - first);
        for (int i = tid; i < count * 2 * N; i += SEL_THREADS) {
            const int t = i / (2 * N), e = i - t * 2 * N;
            sel_cp4(base + i, bc + (size_t)(first + t) * ldbc + e);
        }
        float* per = base + SEL_CHUNK * 2 * N;
        const int c_first = blockIdx.x * cpb;
        const int chans = min(cpb, C - c_first);
        for (int i = tid; i < count * cpb; i += SEL_THREADS) {
            const int t = i / cpb, e = i - t * cpb;
            if (e >= chans) continue;
            const size_t r = (size_t)(first + t);
            sel_cp4(per + i, dt_raw + r * lddt + c_first + e);
            sel_cp4(per + SEL_CHUNK * cpb + i, x + r * ldx + c_first + e);
            sel_cp4(per + 2 * SEL_CHUNK * cpb + i, z + r * ldz + c_first + e);
        }
        sel_commit();
    };

    stage(0, row0);
    int buf = 0;
    for (int first = row0; first < row1; first += SEL_CHUNK, buf ^= 1) {
        sel_wait_all();
        __syncthreads();                              // this chunk has landed; the other buffer's readers are done
        if (first + SEL_CHUNK < row1) stage(buf ^ 1, first + SEL_CHUNK);
        const float* base = sel_smem + buf * buf_floats;
        const float* per = base + SEL_CHUNK * 2 * N;
        const int count = min(SEL_CHUNK, row1 - first);
        for (int t = 0; t < count; t++) {
            const float dt = sel_softplus(per[t * cpb + ch_local]);
            const float xv = per[SEL_CHUNK * cpb + t * cpb + ch_local];
            const float dx = dt * xv;
            const float* Bt = base + t * 2 * N;
            const float* Ct = Bt + N;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < SEL_SLICE; j++) {
                const int n = n0 + j;
                if (n < N) {
                    S[j] = fmaf(expf(dt * A[j]), S[j], dx * Bt[n]);
                    acc = fmaf(S[j], Ct[n], acc);
                }
            }
            for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (sub == 0 && live) {
                const float zv = per[2 * SEL_CHUNK * cpb + t * cpb + ch_local];
                const float out = fmaf(dsk, xv, acc) * (zv / (1.0f + expf(-zv)));
                y[(size_t)(first + t) * C + c] = from_f32<TY>(out);
            }
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < SEL_SLICE; j++)
            if (n0 + j < N) st[n0 + j] = S[j];
    }
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
    int L = 1;
    while (L * SEL_SLICE < N) L <<= 1;
    const int cpb = SEL_THREADS / L;
    const size_t smem = (size_t)2 * SEL_CHUNK * (2 * N + 3 * cpb) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    dim3 grid((C + cpb - 1) / cpb, n_seqs);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(selective_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(selective_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    if (y_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, selective_scan_kernel<bf16>, grid, dim3(SEL_THREADS), smem, stream, x, ldx, dt_raw, lddt,
                       bc, ldbc, z, ldz, a_log, d_skip, state, state_stride, seq_start, seq_slot, (bf16*)y, C, N, L);
    else
        esp_launch_pdl(ESP_PDL_SMALL, selective_scan_kernel<float>, grid, dim3(SEL_THREADS), smem, stream, x, ldx, dt_raw, lddt,
                       bc, ldbc, z, ldz, a_log, d_skip, state, state_stride, seq_start, seq_slot, (float*)y, C, N, L);
    return esp_launch_status();
}
