// Embedding lookup, residual add + RMSNorm, SwiGLU product, finite check and
// the counter-based normal fill used for random weights.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[n, :] = scale * float(table[ids[n], :]); the residual stream is 32-bit in every mode.  ``scale`` is 1 for
// models that feed the table rows as they are (multiplying by 1 changes no bit).
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                                    int n_tokens, int width, int vocab, float scale, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    if (n >= n_tokens) return;
    int id = ids[n];
    if (id < 0 || id >= vocab) {       // never read outside the table
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        id = 0;
    }
    const TW* row = table + (size_t)id * width;
    float* out = x + (size_t)n * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = scale * to_f32(row[i]);
}

ESP_API int esp_embed_gather(const void* table, int table_is_bf16, const int* ids, float* x, int n_tokens, int width,
                             int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (table_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, embed_gather_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)table, ids, x, n_tokens, width, vocab, scale,
                                                                status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, embed_gather_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)table, ids, x, n_tokens, width, vocab, scale,
                                                                 status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- token ids from the last step's choices
// ids[j] = picks[src[j]] where src[j] >= 0: a step that follows a step can take its tokens from the device,
// before the host has seen them.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ picks, const int* __restrict__ src, int n) {
    pdl_trigger();
    pdl_wait();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n && src[j] >= 0) ids[j] = picks[src[j]];
}

ESP_API int esp_feed_tokens(int* ids, const int* picks, const int* src, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    esp_launch_pdl(ESP_PDL_SMALL, feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, picks, src, n);
    return esp_launch_status();
}

// ---------------------------------------------------------------- add + RMSNorm
// Row r works on source row s = rows ? rows[r] : r.
//   v = x[s] + (y ? y[s] * (yscale ? yscale : 1) : 0);  if (write_x) x[s] = v;      (yscale: one factor per channel)
//   h[r] = v * (1 / sqrt(mean(v^2) + eps)) * gamma       (all in 32-bit)
// ``h32`` (may be null) receives the same rows unrounded, for consumers that
// must work from 32-bit values whatever the activation dtype (the router).
// The sum of squares is taken per thread in index order and combined by a
// fixed tree, so a row's result does not depend on the rest of the batch.
template <typename TH>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ yscale,
                                   const float* __restrict__ gamma,
                                   const int* __restrict__ rows, TH* __restrict__ h, float* __restrict__ h32, int width,
                                   float eps, int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * width;
    const float* yr = y ? y + s * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (yr) {
            v += yscale ? yr[i] * yscale[i] : yr[i];
            if (write_x) xr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TH* hr = h + (size_t)r * width;
    float* h32r = h32 ? h32 + (size_t)r * width : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = xr[i];
        if (yr && !write_x) v += yscale ? yr[i] * yscale[i] : yr[i];
        const float o = v * inv * gamma[i];
        hr[i] = from_f32<TH>(o);
        if (h32r) h32r[i] = o;
    }
}

// Same operation for rows whose width is a multiple of 4 and at most 4 * 4 * 1024: each thread keeps up
// to four float4 pieces of the row in registers, so x and y are read once and nothing is read back.
// The sum of squares is taken per thread in piece order and combined by the same fixed tree.
template <typename TH>
__global__ void __launch_bounds__(1024)
add_rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ yscale,
                        const float* __restrict__ gamma, const int* __restrict__ rows, TH* __restrict__ h, float* __restrict__ h32, int width, float eps,
                        int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const int pieces = width / 4;
    float4* xr = reinterpret_cast<float4*>(x + s * width);
    const float4* yr = y ? reinterpret_cast<const float4*>(y + s * width) : nullptr;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            v[i] = xr[q];
            if (yr) {
                float4 a = yr[q];
                if (yscale) {
                    const float4 sc = reinterpret_cast<const float4*>(yscale)[q];
                    a.x *= sc.x; a.y *= sc.y; a.z *= sc.z; a.w *= sc.w;
                }
                v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
                if (write_x) xr[q] = v[i];
            }
            ss = fmaf(v[i].x, v[i].x, ss);
            ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss);
            ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[q];
            const float o0 = v[i].x * inv * gm.x, o1 = v[i].y * inv * gm.y, o2 = v[i].z * inv * gm.z, o3 = v[i].w * inv * gm.w;
            TH* hr = h + (size_t)r * width + 4 * q;
            Vec4<TH>::store(hr, o0, o1, o2, o3);
            if (h32) reinterpret_cast<float4*>(h32 + (size_t)r * width)[q] = make_float4(o0, o1, o2, o3);
        }
    }
}

ESP_API int esp_add_rmsnorm(float* x, const float* y, const float* yscale, const float* gamma, const int* rows, void* h, int h_is_bf16,
                            float* h32, int n_rows, int width, float eps, int write_x, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 4 == 0 && width <= 16384) {
        int threads = ((width / 4 + 3) / 4 + 31) / 32 * 32;       // up to four pieces per thread
        // one piece per thread while a block can hold them: a row's sum then has the same order whatever else is in
        // the step (the 32-bit path relies on it).  Many rows rounded to bfloat16: four pieces per thread, smaller
        // blocks, more rows in flight per SM.
        if (width / 4 <= 1024 && !(h_is_bf16 && n_rows >= 256)) threads = (width / 4 + 31) / 32 * 32;
        if (h_is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y, yscale, gamma, rows, (bf16*)h, h32, width, eps, write_x);
        else
            esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, yscale, gamma, rows, (float*)h, h32, width, eps, write_x);
        return esp_launch_status();
    }
    const int threads = width >= 1024 ? 256 : 128;
    if (h_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y, yscale, gamma, rows, (bf16*)h, h32, width, eps, write_x);
    else
        esp_launch_pdl(ESP_PDL_SMALL, add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, yscale, gamma, rows, (float*)h, h32, width, eps, write_x);
    return esp_launch_status();
}

// ---------------------------------------------------------------- SwiGLU product
// act[m, i] = silu(gu[m, i]) * gu[m, inter + i], gu being [rows, 2*inter] in 32-bit.
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ act, long long rows, int inter) {
    const long long total = rows * inter;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / inter;
        const int i = (int)(idx - m * inter);
        const float g = gu[m * 2 * inter + i];
        const float u = gu[m * 2 * inter + inter + i];
        act[idx] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
    }
}

ESP_API int esp_swiglu(const float* gu, void* act, int act_is_bf16, long long rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long total = rows * inter;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    if (act_is_bf16)
        swiglu_kernel<bf16><<<blocks, 256, 0, stream>>>(gu, (bf16*)act, rows, inter);
    else
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gu, (float*)act, rows, inter);
    return esp_launch_status();
}

// ---------------------------------------------------------------- row gather
// out[r, :] = src[rows[r], :] for bfloat16 rows whose width is a multiple of 8 (16-byte pieces).
__global__ void gather_rows_kernel(const bf16* __restrict__ src, const int* __restrict__ rows, bf16* __restrict__ out,
                                   int n_rows, int pieces) {
    const long long total = (long long)n_rows * pieces;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx / pieces), q = (int)(idx - (long long)r * pieces);
        reinterpret_cast<uint4*>(out)[idx] = reinterpret_cast<const uint4*>(src)[(size_t)rows[r] * pieces + q];
    }
}

ESP_API int esp_gather_rows(const void* src, const int* rows, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width % 8 != 0) return (int)cudaErrorInvalidValue;
    const long long total = (long long)n_rows * (width / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    gather_rows_kernel<<<(int)blocks, 256, 0, stream>>>((const bf16*)src, rows, (bf16*)out, n_rows, width / 8);
    return esp_launch_status();
}

// ---------------------------------------------------------------- finite check
// ORs ``bit`` into *status if any value is a NaN or an infinity.  bfloat16 values are tested on their bits
// (an exponent of all ones), 16 bytes at a time where the count allows.
template <typename T>
__global__ void finite_check_kernel(const T* __restrict__ v, long long count, int* __restrict__ status, int bit) {
    pdl_trigger();
    pdl_wait();
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        bad |= !isfinite(to_f32(v[i]));
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, bit);
}

__global__ void finite_check_bf16x8_kernel(const uint4* __restrict__ v, long long pieces, int* __restrict__ status, int bit) {
    bool bad = false;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pieces; i += (long long)gridDim.x * blockDim.x) {
        const uint4 q = v[i];
        const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; j++)
            bad |= ((w[j] & 0x7F80u) == 0x7F80u) || ((w[j] & 0x7F800000u) == 0x7F800000u);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, bit);
}

ESP_API int esp_finite_check(const void* v, int is_bf16, long long count, int* status, int bit, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (is_bf16) {
        const long long pieces = ((uintptr_t)v & 15) ? 0 : count / 8;
        if (pieces > 0) {
            long long blocks = (pieces + 255) / 256;
            if (blocks > 148 * 16) blocks = 148 * 16;
            finite_check_bf16x8_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4*)v, pieces, status, bit);
        }
        const long long rest = count - pieces * 8;
        if (rest > 0)
            finite_check_kernel<bf16><<<(int)((rest + 255) / 256 > 1184 ? 1184 : (rest + 255) / 256), 256, 0, stream>>>(
                (const bf16*)v + pieces * 8, rest, status, bit);
        return esp_launch_status();
    }
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    esp_launch_pdl(ESP_PDL_SMALL, finite_check_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)v, count, status,
                   bit);
    return esp_launch_status();
}

// ---------------------------------------------------------------- logit soft-cap
// v = cap * tanh(v / cap), in place, for heads that bound their logits this way.
__global__ void softcap_kernel(float* __restrict__ v, long long count, float cap) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        v[i] = cap * tanhf(v[i] / cap);
}

ESP_API int esp_softcap(float* v, long long count, float cap, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    softcap_kernel<<<(int)blocks, 256, 0, stream>>>(v, count, cap);
    return esp_launch_status();
}

// ---------------------------------------------------------------- random normal fill
// value(i) = mean + std * z(i), z from a counter-based generator: two 64-bit
// mixes of (key + i) give two uniforms, Box-Muller gives the normal.  The value
// of an element depends on (key, i) only, not on the launch shape.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void normal_fill_kernel(T* __restrict__ out, long long count, unsigned long long key, float mean, float stddev) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long a = mix64(key + 2ull * (unsigned long long)i);
        const unsigned long long b = mix64(key + 2ull * (unsigned long long)i + 1ull);
        const float u1 = ((float)(a >> 40) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
        const float u2 = (float)(b >> 40) * (1.0f / 16777216.0f);            // [0, 1)
        const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
        out[i] = from_f32<T>(mean + stddev * z);
    }
}

ESP_API int esp_normal_fill(void* out, int out_is_bf16, long long count, unsigned long long key, float mean, float stddev,
                            cudaStream_t stream) {
    if (count <= 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (out_is_bf16)
        normal_fill_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((bf16*)out, count, key, mean, stddev);
    else
        normal_fill_kernel<float><<<(int)blocks, 256, 0, stream>>>((float*)out, count, key, mean, stddev);
    return esp_launch_status();
}

// ---------------------------------------------------------------- depth-weighted average of the layers' results
// history: [slots_of_history, n_rows, width] float; entries 0 .. index hold the results X_0 .. X_index of the
// embedding and the layers so far.  This call finishes layer ``index``:
//   X_(index+1) = x + (y ? y * yscale : 0)        -> history[index + 1]
//   x           = sum_(j = 0 .. index+1) weights[j] * X_j        (added in ascending j)
__global__ void depth_mix_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ yscale,
                                 float* __restrict__ history, const float* __restrict__ weights, int index,
                                 long long count, int width) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (y) v += yscale ? y[i] * yscale[i % width] : y[i];
        history[(size_t)(index + 1) * count + i] = v;
        float acc = 0.f;
        for (int j = 0; j <= index; j++) acc = fmaf(weights[j], history[(size_t)j * count + i], acc);
        x[i] = fmaf(weights[index + 1], v, acc);
    }
}

ESP_API int esp_depth_mix(float* x, const float* y, const float* yscale, float* history, const float* weights, int index,
                          int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const long long count = (long long)n_rows * width;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    esp_launch_pdl(ESP_PDL_SMALL, depth_mix_kernel, dim3((int)blocks), dim3(256), 0, stream, x, y, yscale, history, weights,
                   index, count, width);
    return esp_launch_status();
}

// ---------------------------------------------------------------- xIELU
// act = a_p z^2 + z / 2 (z > 0);  a_n (exp(z) - 1 - z) + z / 2 (z <= 0);  a_p = softplus(p), a_n = 1/2 + softplus(q),
// p and q being the two learned numbers in ``pq``.
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename TO>
__global__ void xielu_kernel(const float* __restrict__ z, const float* __restrict__ pq, TO* __restrict__ act, long long count) {
    pdl_trigger();
    pdl_wait();
    const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
    auto f = [&](float v) { return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v); };
    if (count % 4 == 0 && ((size_t)z % 16) == 0 && ((size_t)act % 16) == 0) {       // four values a piece
        const long long pieces = count / 4;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pieces; i += (long long)gridDim.x * blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(z)[i];
            Vec4<TO>::store(act + 4 * i, f(v.x), f(v.y), f(v.z), f(v.w));
        }
        return;
    }
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        act[i] = from_f32<TO>(f(z[i]));
}

ESP_API int esp_xielu(const float* z, const float* pq, void* act, int act_is_bf16, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, xielu_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, z, pq, (bf16*)act, count);
    else
        esp_launch_pdl(ESP_PDL_SMALL, xielu_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, pq, (float*)act, count);
    return esp_launch_status();
}

// out = tanh(in), for the small hidden layer of a data-dependent decay
template <typename TO>
__global__ void tanh_kernel(const float* __restrict__ z, TO* __restrict__ out, long long count) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(tanhf(z[i]));
}

ESP_API int esp_tanh(const float* z, void* out, int out_is_bf16, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, tanh_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, z, (bf16*)out, count);
    else
        esp_launch_pdl(ESP_PDL_SMALL, tanh_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, (float*)out, count);
    return esp_launch_status();
}

// ---------------------------------------------------------------- summed embeddings
// x[n] = table[id] + bigram[row] + position vector.  row = (prev * mul_prev + id * mul_cur) mod buckets, prev being
// the token before this one in its sequence; a sequence's first token reads row ``buckets``.  The token before a
// run's first token is the sequence's state (prev_state[slot] holds token + 1; 0: the sequence has no token yet);
// the block of a run's first token also leaves the run's last token there.  Position vector: entry 2i is
// sin(p * freq[i]), entry 2i + 1 its cosine, the angle taken in 32-bit.  ``bigram`` and ``freq`` may be null.
template <typename TW>
__global__ void embed_sum_kernel(const TW* __restrict__ table, const TW* __restrict__ bigram, const float* __restrict__ freq,
                                 const int* __restrict__ ids, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                 int* __restrict__ prev_state, float* __restrict__ x, int width, int vocab, int buckets,
                                 long long mul_prev, long long mul_cur, float scale, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        id = 0;
    }
    const int seq = tok_seq[n];
    const bool first = n == seq_start[seq];
    const TW* brow = nullptr;
    if (bigram) {
        int prev;
        if (first) {
            prev = prev_state[seq_slot[seq]] - 1;
        } else {
            prev = ids[n - 1];
            if (prev < 0 || prev >= vocab) prev = 0;
        }
        const long long row = prev < 0 ? (long long)buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        brow = bigram + (size_t)row * width;
    }
    const TW* row = table + (size_t)id * width;
    const float p = (float)tok_pos[n];
    float* out = x + (size_t)n * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = scale * to_f32(row[i]);
        if (brow) v += to_f32(brow[i]);
        if (freq) {
            const float a = p * freq[i >> 1];
            v += (i & 1) ? cosf(a) : sinf(a);
        }
        out[i] = v;
    }
    if (first && bigram) {
        __syncthreads();                       // the state was read by thread-private code above; one thread writes it
        if (threadIdx.x == 0) {
            int last = ids[seq_start[seq + 1] - 1];
            if (last < 0 || last >= vocab) last = 0;
            prev_state[seq_slot[seq]] = last + 1;
        }
    }
}

ESP_API int esp_embed_sum(const void* table, const void* bigram, int table_is_bf16, const float* freq, const int* ids,
                          const int* tok_seq, const int* tok_pos, const int* seq_start, const int* seq_slot, int* prev_state,
                          float* x, int n_tokens, int width, int vocab, int buckets, long long mul_prev, long long mul_cur,
                          float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (bigram && (!prev_state || buckets <= 0)) return (int)cudaErrorInvalidValue;
    if (table_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, embed_sum_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)table,
                       (const bf16*)bigram, freq, ids, tok_seq, tok_pos, seq_start, seq_slot, prev_state, x, width, vocab,
                       buckets, mul_prev, mul_cur, scale, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, embed_sum_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)table,
                       (const float*)bigram, freq, ids, tok_seq, tok_pos, seq_start, seq_slot, prev_state, x, width, vocab,
                       buckets, mul_prev, mul_cur, scale, status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- norm of a sublayer's result + add + the next norm
// Row r works on source row s = rows ? rows[r] : r.
//   d = y[s] / sqrt(mean(y[s]^2) + eps_y) * gamma_y;  v = x[s] + d;  if (write_x) x[s] = v;
//   h[r] = v / sqrt(mean(v^2) + eps) * gamma     (h null: only the first two lines)
// All in 32-bit; sums of squares per thread in index order, combined by a fixed tree.  With ``x`` null the kernel
// writes d itself to ``h32`` (the normed result alone).
template <typename TH>
__global__ void norm_add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma_y,
                                        float eps_y, const float* __restrict__ gamma, const int* __restrict__ rows,
                                        TH* __restrict__ h, float* __restrict__ h32, int width, float eps, int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const float* yr = y + s * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
    const float inv_y = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps_y);
    if (!x) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) h32[(size_t)r * width + i] = yr[i] * inv_y * gamma_y[i];
        return;
    }
    float* xr = x + s * width;
    ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i] + yr[i] * inv_y * gamma_y[i];
        if (write_x) xr[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!h) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    TH* hr = h + (size_t)r * width;
    float* h32r = h32 ? h32 + (size_t)r * width : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = write_x ? xr[i] : xr[i] + yr[i] * inv_y * gamma_y[i];
        const float o = v * inv * gamma[i];
        hr[i] = from_f32<TH>(o);
        if (h32r) h32r[i] = o;
    }
}

// Same operation for rows whose width is a multiple of 4 and at most 4 * 4 * 1024: each thread keeps up to four
// float4 pieces of y and of x in registers, so both are read once.  Sums of squares per thread in piece order,
// combined by the same fixed tree.  (x given; h may be null.)
template <typename TH>
__global__ void __launch_bounds__(1024)
norm_add_rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma_y,
                             float eps_y, const float* __restrict__ gamma, const int* __restrict__ rows,
                             TH* __restrict__ h, float* __restrict__ h32, int width, float eps, int write_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const int pieces = width / 4;
    float4* xr = reinterpret_cast<float4*>(x + s * width);
    const float4* yr = reinterpret_cast<const float4*>(y + s * width);
    float4 v[4], a[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            a[i] = yr[q];
            v[i] = xr[q];
            ss = fmaf(a[i].x, a[i].x, ss);
            ss = fmaf(a[i].y, a[i].y, ss);
            ss = fmaf(a[i].z, a[i].z, ss);
            ss = fmaf(a[i].w, a[i].w, ss);
        }
    }
    const float inv_y = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps_y);
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            const float4 gy = reinterpret_cast<const float4*>(gamma_y)[q];
            v[i].x += a[i].x * inv_y * gy.x; v[i].y += a[i].y * inv_y * gy.y;
            v[i].z += a[i].z * inv_y * gy.z; v[i].w += a[i].w * inv_y * gy.w;
            if (write_x) xr[q] = v[i];
            ss = fmaf(v[i].x, v[i].x, ss);
            ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss);
            ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    if (!h) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < pieces) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[q];
            const float o0 = v[i].x * inv * gm.x, o1 = v[i].y * inv * gm.y, o2 = v[i].z * inv * gm.z, o3 = v[i].w * inv * gm.w;
            Vec4<TH>::store(h + (size_t)r * width + 4 * q, o0, o1, o2, o3);
            if (h32) reinterpret_cast<float4*>(h32 + (size_t)r * width)[q] = make_float4(o0, o1, o2, o3);
        }
    }
}

ESP_API int esp_norm_add_rmsnorm(float* x, const float* y, const float* gamma_y, float eps_y, const float* gamma,
                                 const int* rows, void* h, int h_is_bf16, float* h32, int n_rows, int width, float eps,
                                 int write_x, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!y || !gamma_y || (!x && !h32) || (h && !gamma)) return (int)cudaErrorInvalidValue;
    if (x && width % 4 == 0 && width <= 16384) {
        // one piece per thread while a block can hold them (the thread count depends on the width alone in the 32-bit
        // path, so a row's sums have one order whatever else is in the step); many rows rounded to bfloat16: four
        // pieces per thread, smaller blocks, more rows in flight per SM
        int threads = ((width / 4 + 3) / 4 + 31) / 32 * 32;
        if (width / 4 <= 1024 && !(h_is_bf16 && n_rows >= 256)) threads = (width / 4 + 31) / 32 * 32;
        if (h_is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, norm_add_rmsnorm_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y,
                           gamma_y, eps_y, gamma, rows, (bf16*)h, h32, width, eps, write_x);
        else
            esp_launch_pdl(ESP_PDL_SMALL, norm_add_rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y,
                           gamma_y, eps_y, gamma, rows, (float*)h, h32, width, eps, write_x);
        return esp_launch_status();
    }
    const int threads = width >= 2048 ? 512 : width >= 512 ? 256 : 128;
    if (h_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, norm_add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma_y,
                       eps_y, gamma, rows, (bf16*)h, h32, width, eps, write_x);
    else
        esp_launch_pdl(ESP_PDL_SMALL, norm_add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, y, gamma_y,
                       eps_y, gamma, rows, (float*)h, h32, width, eps, write_x);
    return esp_launch_status();
}

// ---------------------------------------------------------------- squared ReLU
// act[m, i] = max(z[m, i] * (row_scale ? row_scale[m] : 1), 0)^2
template <typename TO>
__global__ void relu2_kernel(const float* __restrict__ z, const float* __restrict__ row_scale, TO* __restrict__ act,
                             long long rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * width;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float v = z[i];
        if (row_scale) v *= row_scale[i / width];
        v = fmaxf(v, 0.f);
        act[i] = from_f32<TO>(v * v);
    }
}

ESP_API int esp_relu2(const float* z, const float* row_scale, void* act, int act_is_bf16, long long rows, int width,
                      cudaStream_t stream) {
    if (rows <= 0) return 0;
    long long blocks = (rows * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, relu2_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, z, row_scale, (bf16*)act, rows, width);
    else
        esp_launch_pdl(ESP_PDL_SMALL, relu2_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, row_scale, (float*)act, rows, width);
    return esp_launch_status();
}

// ---------------------------------------------------------------- hyper-connections
// A layer over S copies of the residual stream, streams[s, row, :] (float).  One launch does, for every row it is
// given, what lies between two sublayers:
//   1. (y given) the write of the sublayer that has just run, all copies at once from the old ones:
//          new_t = sum_s mix[s, t] old_s + out_w[t] y            (old_s = x0 for every s when x0 is given: the copies
//                                                                  of a stack's first layer all equal what enters it)
//   2. the read of the sublayer that comes next: u = sum_s read_w[s] new_s (read_w null: the plain sum, which is what
//      leaves the stack), h = u / sqrt(mean(u^2) + eps) * gamma in the activation dtype, u itself to u_out.
// ``rows`` selects the rows (the model's last norm wants a few); with write_streams 0 the copies are left as they are.
// Every sum runs in ascending s, a row's sum of squares over a block of fixed size: a row's result depends on the row
// alone.  A thread owns its channels in both passes, so it may overwrite the copies in the second.
constexpr int HC_MAX_STREAMS = 8;

template <typename T>
__global__ void hc_step_kernel(float* __restrict__ streams, const float* __restrict__ x0, const float* __restrict__ y,
                               const float* __restrict__ mix, const float* __restrict__ out_w,
                               const float* __restrict__ read_w, const float* __restrict__ gamma,
                               const int* __restrict__ rows, T* __restrict__ h, float* __restrict__ u_out, int S,
                               long long stream_stride, int width, float eps, int write_streams) {
    pdl_trigger();
    __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_out[HC_MAX_STREAMS], s_read[HC_MAX_STREAMS];
    __shared__ float scratch[33];
    const int tid = threadIdx.x;
    if (tid < S * S) s_mix[tid] = mix ? mix[tid] : (tid / S == tid % S ? 1.f : 0.f);
    if (tid < S) {
        s_out[tid] = out_w ? out_w[tid] : 0.f;
        s_read[tid] = read_w ? read_w[tid] : 1.f;
    }
    __syncthreads();
    pdl_wait();
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const float* yrow = y ? y + r * width : nullptr;
    const float* x0row = x0 ? x0 + r * width : nullptr;
    float* srow = streams + r * width;
    float ss = 0.f;
    for (int pass = 0; pass < 2; pass++) {
        if (pass == 1 && !write_streams && !h && !u_out) break;
        float inv = 0.f;
        if (pass == 1) inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int d = tid; d < width; d += blockDim.x) {
            float old[HC_MAX_STREAMS], now[HC_MAX_STREAMS];
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; s++)
                if (s < S) old[s] = x0row ? x0row[d] : srow[(size_t)s * stream_stride + d];
            if (yrow) {
                const float yv = yrow[d];
#pragma unroll
                for (int t = 0; t < HC_MAX_STREAMS; t++) {
                    if (t >= S) break;
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; s++)
                        if (s < S) a = fmaf(s_mix[s * S + t], old[s], a);
                    now[t] = fmaf(s_out[t], yv, a);
                }
            } else {
#pragma unroll
                for (int s = 0; s < HC_MAX_STREAMS; s++)
                    if (s < S) now[s] = old[s];
            }
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; s++)
                if (s < S) u = fmaf(s_read[s], now[s], u);
            if (pass == 0) {
                ss = fmaf(u, u, ss);
            } else {
                if (write_streams && (yrow || x0row)) {
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; s++)
                        if (s < S) srow[(size_t)s * stream_stride + d] = now[s];
                }
                if (u_out) u_out[r * width + d] = u;
                if (h) h[(size_t)i * width + d] = from_f32<T>(u * inv * gamma[d]);
            }
        }
    }
}

// The same step for S known at compile time and rows whose pieces of four channels are aligned: a thread owns pieces
// of four channels, every copy arrives as one 16-byte load, and the loops over the copies are unrolled, so a block needs
// few registers and several are resident.  Per element the arithmetic and its order are those of the kernel above.
template <typename T, int S>
__global__ void __launch_bounds__(256)
hc_step_vec_kernel(float* __restrict__ streams, const float* __restrict__ x0, const float* __restrict__ y,
                   const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ read_w,
                   const float* __restrict__ gamma, const int* __restrict__ rows, T* __restrict__ h,
                   float* __restrict__ u_out, long long stream_stride, int width, float eps, int write_streams) {
    pdl_trigger();
    __shared__ float scratch[33];
    float m[S * S], ow[S], rw[S];
#pragma unroll
    for (int i = 0; i < S * S; i++) m[i] = mix ? mix[i] : (i / S == i % S ? 1.f : 0.f);
#pragma unroll
    for (int s = 0; s < S; s++) {
        ow[s] = out_w ? out_w[s] : 0.f;
        rw[s] = read_w ? read_w[s] : 1.f;
    }
    pdl_wait();
    const int i = blockIdx.x, tid = threadIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const float* yrow = y ? y + r * width : nullptr;
    const float* x0row = x0 ? x0 + r * width : nullptr;
    float* srow = streams + r * width;
    float ss = 0.f;
    for (int pass = 0; pass < 2; pass++) {
        if (pass == 1 && !write_streams && !h && !u_out) break;
        float inv = 0.f;
        if (pass == 1) inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int d = 4 * tid; d < width; d += 4 * blockDim.x) {
            float now[S][4];
            {
                float old[S][4];
#pragma unroll
                for (int s = 0; s < S; s++) {
                    const float4 v = *reinterpret_cast<const float4*>(x0row ? x0row + d : srow + (size_t)s * stream_stride + d);
                    old[s][0] = v.x, old[s][1] = v.y, old[s][2] = v.z, old[s][3] = v.w;
                }
                if (yrow) {
                    const float4 y4 = *reinterpret_cast<const float4*>(yrow + d);
                    const float yv[4] = {y4.x, y4.y, y4.z, y4.w};
#pragma unroll
                    for (int t = 0; t < S; t++)
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float a = 0.f;
#pragma unroll
                            for (int s = 0; s < S; s++) a = fmaf(m[s * S + t], old[s][e], a);
                            now[t][e] = fmaf(ow[t], yv[e], a);
                        }
                } else {
#pragma unroll
                    for (int s = 0; s < S; s++)
#pragma unroll
                        for (int e = 0; e < 4; e++) now[s][e] = old[s][e];
                }
            }
            float u[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < S; s++) a = fmaf(rw[s], now[s][e], a);
                u[e] = a;
            }
            if (pass == 0) {
#pragma unroll
                for (int e = 0; e < 4; e++) ss = fmaf(u[e], u[e], ss);
            } else {
                if (write_streams && (yrow || x0row)) {
#pragma unroll
                    for (int s = 0; s < S; s++)
                        *reinterpret_cast<float4*>(srow + (size_t)s * stream_stride + d) =
                            make_float4(now[s][0], now[s][1], now[s][2], now[s][3]);
                }
                if (u_out) *reinterpret_cast<float4*>(u_out + r * width + d) = make_float4(u[0], u[1], u[2], u[3]);
                if (h) {
                    const float4 g = *reinterpret_cast<const float4*>(gamma + d);
                    Vec4<T>::store(h + (size_t)i * width + d, u[0] * inv * g.x, u[1] * inv * g.y, u[2] * inv * g.z,
                                   u[3] * inv * g.w);
                }
            }
        }
    }
}

template <typename T, int S>
static void hc_step_vec_launch(float* streams, const float* x0, const float* y, const float* mix, const float* out_w,
                               const float* read_w, const float* gamma, const int* rows, T* h, float* u_out,
                               long long stream_stride, int n_rows, int width, float eps, int write_streams,
                               cudaStream_t stream) {
    const int threads = width >= 2048 ? 256 : (width >= 512 ? 128 : 64);
    esp_launch_pdl(ESP_PDL_SMALL, hc_step_vec_kernel<T, S>, dim3(n_rows), dim3(threads), 0, stream, streams, x0, y, mix, out_w,
                   read_w, gamma, rows, h, u_out, stream_stride, width, eps, write_streams);
}

template <typename T>
static bool hc_step_vec(float* streams, const float* x0, const float* y, const float* mix, const float* out_w,
                        const float* read_w, const float* gamma, const int* rows, T* h, float* u_out, int S,
                        long long stream_stride, int n_rows, int width, float eps, int write_streams, cudaStream_t stream) {
    const size_t all = (size_t)streams | (size_t)x0 | (size_t)y | (size_t)gamma | (size_t)h | (size_t)u_out;
    if (S > 4 || width % 4 || stream_stride % 4 || (all & 15)) return false;
#define ESP_HC_VEC(N)                                                                                                   \
    hc_step_vec_launch<T, N>(streams, x0, y, mix, out_w, read_w, gamma, rows, h, u_out, stream_stride, n_rows, width, \
                             eps, write_streams, stream)
    if (S == 1) ESP_HC_VEC(1);
    else if (S == 2) ESP_HC_VEC(2);
    else if (S == 3) ESP_HC_VEC(3);
    else ESP_HC_VEC(4);
#undef ESP_HC_VEC
    return true;
}

ESP_API int esp_hc_step(float* streams, const float* x0, const float* y, const float* mix, const float* out_w,
                        const float* read_w, const float* gamma, const int* rows, void* h, int h_is_bf16, float* u_out,
                        int n_streams, long long stream_stride, int n_rows, int width, float eps, int write_streams,
                        cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > HC_MAX_STREAMS || width <= 0 || (h && !gamma)) return (int)cudaErrorInvalidValue;
    // which form runs depends on the sizes and the buffers' alignment alone, never on the rows of a step
    if (h_is_bf16 ? hc_step_vec<bf16>(streams, x0, y, mix, out_w, read_w, gamma, rows, (bf16*)h, u_out, n_streams, stream_stride,
                                      n_rows, width, eps, write_streams, stream)
                  : hc_step_vec<float>(streams, x0, y, mix, out_w, read_w, gamma, rows, (float*)h, u_out, n_streams,
                                       stream_stride, n_rows, width, eps, write_streams, stream))
        return esp_launch_status();
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (h_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, hc_step_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, streams, x0, y, mix, out_w,
                       read_w, gamma, rows, (bf16*)h, u_out, n_streams, stream_stride, width, eps, write_streams);
    else
        esp_launch_pdl(ESP_PDL_SMALL, hc_step_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, streams, x0, y, mix, out_w,
                       read_w, gamma, rows, (float*)h, u_out, n_streams, stream_stride, width, eps, write_streams);
    return esp_launch_status();
}

// ---------------------------------------------------------------- gated unit with clamped branches
// act[m, i] = g sigmoid(alpha g) (u + shift) with g = min(gu[m, i], limit), u = clamp(gu[m, inter + i], -limit, limit);
// gu is [rows, 2 * inter] in 32-bit.
template <typename TO>
__global__ void glu_clamped_kernel(const float* __restrict__ gu, TO* __restrict__ act, long long rows, int inter, float limit,
                                   float alpha, float shift) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * inter;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / inter;
        const int i = (int)(idx - m * inter);
        const float g = fminf(gu[m * 2 * inter + i], limit);
        const float u = fminf(fmaxf(gu[m * 2 * inter + inter + i], -limit), limit);
        act[idx] = from_f32<TO>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

// The same for widths of whole pieces of four channels: a thread takes four neighbours of gate and of up in one 16-byte
// load each; per element the arithmetic is that of the kernel above.
template <typename TO>
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(const float* __restrict__ gu, TO* __restrict__ act, long long rows, int inter, float limit,
                       float alpha, float shift) {
    pdl_trigger();
    pdl_wait();
    const int quads = inter / 4;
    const long long total = rows * quads;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / quads;
        const int i = 4 * (int)(idx - m * quads);
        const float4 g4 = *reinterpret_cast<const float4*>(gu + m * 2 * inter + i);
        const float4 u4 = *reinterpret_cast<const float4*>(gu + m * 2 * inter + inter + i);
        const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float g = fminf(gs[e], limit);
            const float u = fminf(fmaxf(us[e], -limit), limit);
            r[e] = g / (1.0f + expf(-alpha * g)) * (u + shift);
        }
        Vec4<TO>::store(act + m * inter + i, r[0], r[1], r[2], r[3]);
    }
}

ESP_API int esp_glu_clamped(const float* gu, void* act, int act_is_bf16, long long rows, int inter, float limit, float alpha,
                            float shift, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter % 4 == 0 && (((size_t)gu | (size_t)act) & 15) == 0) {
        const long long total = rows * (inter / 4);
        const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
        if (act_is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, glu_clamped_vec_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, gu, (bf16*)act, rows, inter, limit, alpha, shift);
        else
            esp_launch_pdl(ESP_PDL_SMALL, glu_clamped_vec_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float*)act, rows, inter, limit, alpha, shift);
        return esp_launch_status();
    }
    const long long total = rows * inter;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    if (act_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, glu_clamped_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, gu, (bf16*)act, rows, inter, limit, alpha, shift);
    else
        esp_launch_pdl(ESP_PDL_SMALL, glu_clamped_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float*)act, rows, inter, limit, alpha, shift);
    return esp_launch_status();
}

// ---------------------------------------------------------------- small helpers of composite mixers
// out = sum_i scale[i] * src[i] over up to four float arrays of ``count`` values, added in the order given.
__global__ void weighted_sum_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                    const float* __restrict__ c, const float* __restrict__ d, float sa, float sb, float sc,
                                    float sd, long long count) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        float v = sa * a[i];
        if (b) v = fmaf(sb, b[i], v);
        if (c) v = fmaf(sc, c[i], v);
        if (d) v = fmaf(sd, d[i], v);
        out[i] = v;
    }
}

// The same, four neighbours a thread (the sum of an element is formed in the same order).
__global__ void __launch_bounds__(256)
weighted_sum_vec_kernel(float4* __restrict__ out, const float4* __restrict__ a, const float4* __restrict__ b,
                        const float4* __restrict__ c, const float4* __restrict__ d, float sa, float sb, float sc, float sd,
                        long long quads) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < quads; i += (long long)gridDim.x * blockDim.x) {
        const float4 x = a[i];
        float4 v = make_float4(sa * x.x, sa * x.y, sa * x.z, sa * x.w);
        if (b) { const float4 t = b[i]; v.x = fmaf(sb, t.x, v.x), v.y = fmaf(sb, t.y, v.y), v.z = fmaf(sb, t.z, v.z), v.w = fmaf(sb, t.w, v.w); }
        if (c) { const float4 t = c[i]; v.x = fmaf(sc, t.x, v.x), v.y = fmaf(sc, t.y, v.y), v.z = fmaf(sc, t.z, v.z), v.w = fmaf(sc, t.w, v.w); }
        if (d) { const float4 t = d[i]; v.x = fmaf(sd, t.x, v.x), v.y = fmaf(sd, t.y, v.y), v.z = fmaf(sd, t.z, v.z), v.w = fmaf(sd, t.w, v.w); }
        out[i] = v;
    }
}

ESP_API int esp_weighted_sum(float* out, const float* a, const float* b, const float* c, const float* d, float sa, float sb,
                             float sc, float sd, long long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (!a) return (int)cudaErrorInvalidValue;
    if (count % 4 == 0 && (((size_t)out | (size_t)a | (size_t)b | (size_t)c | (size_t)d) & 15) == 0) {
        const long long quads = count / 4;
        long long vb = (quads + 255) / 256;
        if (vb > 148 * 16) vb = 148 * 16;
        esp_launch_pdl(ESP_PDL_SMALL, weighted_sum_vec_kernel, dim3((int)vb), dim3(256), 0, stream, (float4*)out, (const float4*)a,
                       (const float4*)b, (const float4*)c, (const float4*)d, sa, sb, sc, sd, quads);
        return esp_launch_status();
    }
    long long blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    esp_launch_pdl(ESP_PDL_SMALL, weighted_sum_kernel, dim3((int)blocks), dim3(256), 0, stream, out, a, b, c, d, sa, sb, sc, sd, count);
    return esp_launch_status();
}

// dst[r, :] = src[r, c0 : c0 + width] in the activation dtype (src float with row stride ld).
template <typename TO>
__global__ void cast_cols_kernel(const float* __restrict__ src, long long ld, TO* __restrict__ dst, long long rows, int width) {
    pdl_trigger();
    pdl_wait();
    const long long total = rows * width;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        dst[i] = from_f32<TO>(src[r * ld + (i - r * width)]);
    }
}

ESP_API int esp_cast_cols(const float* src, long long ld, void* dst, int dst_is_bf16, long long rows, int width,
                          cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    long long blocks = (rows * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dst_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, cast_cols_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, src, ld, (bf16*)dst, rows, width);
    else
        esp_launch_pdl(ESP_PDL_SMALL, cast_cols_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, src, ld, (float*)dst, rows, width);
    return esp_launch_status();
}
