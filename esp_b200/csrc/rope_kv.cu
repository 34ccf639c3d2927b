// Rotary position encoding (split-half) of the new queries and keys in 32-bit,
// and the write of the new keys and values into the paged cache.
//
// qkv: [n_tokens, (nh + 2*nkv) * hd] float; ``bias`` (same width, may be null) is
// added first.  Head h of the
// query block is columns [h*hd, (h+1)*hd); keys follow the queries, values the
// keys.  For i < rot/2 and the token's absolute position p:
//   o[i]         = x[i] * cos[p][i] - x[i + rot/2] * sin[p][i]
//   o[i + rot/2] = x[i + rot/2] * cos[p][i] + x[i] * sin[p][i]
// Columns at or beyond ``rot`` pass through (rot = 0: no rotation at all).
// Keys are cached after rotation.  A page holds PAGE consecutive positions of
// one sequence: K/V are [pages, nkv, PAGE, hd]; the page of position p is
// block_table[seq * table_stride + p / PAGE].
#include "common.cuh"

template <typename T>
__global__ void rope_kvwrite_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                    const int* __restrict__ tok_seq,
                                    const int* __restrict__ tok_pos, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, int rot, int max_pos, T* __restrict__ q_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                                    int table_stride, int n_pages, int page, int nh, int nkv, int hd, int write_kv,
                                    int heads_per_block, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int pos = tok_pos[n];
    const int seq = tok_seq[n];
    const int half = rot / 2;
    const int width = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)n * width;
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const int heads = nh + 2 * nkv;
    const int head_lo = blockIdx.y * heads_per_block, head_hi = min(heads, head_lo + heads_per_block);
    for (int idx = threadIdx.x; idx < (head_hi - head_lo) * hd; idx += blockDim.x) {
        const int head = head_lo + idx / hd, i = idx % hd;
        const float* x = src + (size_t)head * hd;
        const float* b = bias ? bias + (size_t)head * hd : nullptr;
        float v = x[i] + (b ? b[i] : 0.f);
        if (head < nh + nkv && i < rot) {          // queries and keys rotate, values do not
            if (i < half) {
                const float other = x[i + half] + (b ? b[i + half] : 0.f);
                v = v * cs[i] - other * sn[i];
            } else {
                const float other = x[i - half] + (b ? b[i - half] : 0.f);
                v = v * cs[i - half] + other * sn[i - half];
            }
        }
        if (head < nh) {
            q_out[((size_t)n * nh + head) * hd + i] = from_f32<T>(v);
        } else if (page_id >= 0) {
            const bool is_k = head < nh + nkv;
            const int kvh = is_k ? head - nh : head - nh - nkv;
            T* dst = (is_k ? k_cache : v_cache) + (((size_t)page_id * nkv + kvh) * page + in_page) * hd + i;
            *dst = from_f32<T>(v);
        }
    }
}

// The same for full rotation (rot == hd, hd a multiple of 8) with 16-byte accesses: a thread owns four
// consecutive pairs (i, i + hd/2) of one head of one token.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kvwrite_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, const int* __restrict__ tok_seq,
                        const int* __restrict__ tok_pos, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        int max_pos, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_stride, int n_pages, int page, int nh, int nkv,
                        int hd, int write_kv, int heads_per_block, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int pos = tok_pos[n], seq = tok_seq[n];
    const int half = hd / 2, quads = half / 4, heads = nh + 2 * nkv;
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const float* src = qkv + (size_t)n * heads * hd;
    const float4* cs = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half);
    const float4* sn = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half);
    const int head_lo = blockIdx.y * heads_per_block, head_hi = min(heads, head_lo + heads_per_block);
    for (int idx = threadIdx.x; idx < (head_hi - head_lo) * quads; idx += blockDim.x) {
        const int head = head_lo + idx / quads, qd = idx % quads, i0 = qd * 4;
        const float* x = src + (size_t)head * hd;
        float4 lo = *reinterpret_cast<const float4*>(x + i0), hi = *reinterpret_cast<const float4*>(x + i0 + half);
        if (bias) {
            const float4 bl = *reinterpret_cast<const float4*>(bias + (size_t)head * hd + i0);
            const float4 bh = *reinterpret_cast<const float4*>(bias + (size_t)head * hd + i0 + half);
            lo.x += bl.x; lo.y += bl.y; lo.z += bl.z; lo.w += bl.w;
            hi.x += bh.x; hi.y += bh.y; hi.z += bh.z; hi.w += bh.w;
        }
        float4 ol = lo, oh = hi;
        if (head < nh + nkv) {                       // queries and keys rotate, values do not
            const float4 c = cs[qd], s = sn[qd];
            ol.x = lo.x * c.x - hi.x * s.x; oh.x = hi.x * c.x + lo.x * s.x;
            ol.y = lo.y * c.y - hi.y * s.y; oh.y = hi.y * c.y + lo.y * s.y;
            ol.z = lo.z * c.z - hi.z * s.z; oh.z = hi.z * c.z + lo.z * s.z;
            ol.w = lo.w * c.w - hi.w * s.w; oh.w = hi.w * c.w + lo.w * s.w;
        }
        T* dst = nullptr;
        if (head < nh) {
            dst = q_out + ((size_t)n * nh + head) * hd;
        } else if (page_id >= 0) {
            const bool is_k = head < nh + nkv;
            const int kvh = is_k ? head - nh : head - nh - nkv;
            dst = (is_k ? k_cache : v_cache) + (((size_t)page_id * nkv + kvh) * page + in_page) * hd;
        }
        if (dst) {
            Vec4<T>::store(dst + i0, ol.x, ol.y, ol.z, ol.w);
            Vec4<T>::store(dst + i0 + half, oh.x, oh.y, oh.z, oh.w);
        }
    }
}

ESP_API int esp_rope_kvwrite(const float* qkv, const float* bias, const int* tok_seq, const int* tok_pos, const float* cos_t,
                             const float* sin_t, int rot, int max_pos, void* q_out, void* k_cache, void* v_cache,
                             int is_bf16, const int* block_table, int table_stride, int n_pages, int page, int n_tokens,
                             int nh, int nkv, int hd, int write_kv, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1) || nh + 2 * nkv > 65535) return (int)cudaErrorInvalidValue;
    // few tokens (decode): one head per block keeps every load in flight at once; many tokens: eight heads
    // per block keep the number of blocks down
    if (rot == hd && hd % 8 == 0 && cos_t && n_tokens > 64) {
        // many tokens, full rotation: the 16-byte version, 64 heads per block (several pieces in flight per thread)
        const int hpb = 64;
        const dim3 vgrid(n_tokens, (nh + 2 * nkv + hpb - 1) / hpb);
        if (is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_vec_kernel<bf16>, dim3(vgrid), dim3(256), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, max_pos,
                                                                    (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache,
                                                                    block_table, table_stride, n_pages, page, nh, nkv, hd,
                                                                    write_kv, hpb, status);
        else
            esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_vec_kernel<float>, dim3(vgrid), dim3(256), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, max_pos,
                                                                     (float*)q_out, (float*)k_cache, (float*)v_cache,
                                                                     block_table, table_stride, n_pages, page, nh, nkv,
                                                                     hd, write_kv, hpb, status);
        return esp_launch_status();
    }
    const int heads_per_block = n_tokens <= 64 ? 1 : 8;
    const dim3 grid(n_tokens, (nh + 2 * nkv + heads_per_block - 1) / heads_per_block);
    const int threads = heads_per_block == 1 ? (hd >= 128 ? 128 : (hd + 31) / 32 * 32) : 256;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_kernel<bf16>, dim3(grid), dim3(threads), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, rot, max_pos,
                                                               (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, block_table,
                                                               table_stride, n_pages, page, nh, nkv, hd, write_kv, heads_per_block, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, rope_kvwrite_kernel<float>, dim3(grid), dim3(threads), 0, stream, qkv, bias, tok_seq, tok_pos, cos_t, sin_t, rot, max_pos,
                                                                (float*)q_out, (float*)k_cache, (float*)v_cache,
                                                                block_table, table_stride, n_pages, page, nh, nkv, hd,
                                                                write_kv, heads_per_block, status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- queries and keys with a norm per head, no rotation
// qkv: [n_tokens, nh*hd + nkv*hd + nkv*vd] float; ``bias`` (same width, may be null) is added first.  Every query
// and key head is divided by its root mean square (eps inside the root) and multiplied by a weight vector of hd
// numbers that all heads share (q_w, k_w; null: no norm for that side).  Queries are then multiplied by
// 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1), p the token's position (temp_every 0: no such factor).
// Keys [pages, nkv, PAGE, hd] and values [pages, nkv, PAGE, vd] go to the token's place in the paged cache.
// One warp per head; everything in 32-bit.
template <typename T>
__global__ void qknorm_kvwrite_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                      const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                      float temp_coef, int temp_every, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_cache,
                                      T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                                      int n_pages, int page, int nh, int nkv, int hd, int vd, int write_kv,
                                      int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int pos = tok_pos[n], seq = tok_seq[n];
    const size_t width = (size_t)(nh + nkv) * hd + (size_t)nkv * vd;
    const float* src = qkv + (size_t)n * width;
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    float q_factor = 1.0f;
    if (temp_every > 0) q_factor = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    for (int head = warp; head < nh + 2 * nkv; head += nwarp) {
        if (head < nh + nkv) {
            const float* x = src + (size_t)head * hd;
            const float* b = bias ? bias + (size_t)head * hd : nullptr;
            const float* w = head < nh ? q_w : k_w;
            float ss = 0.f;
            for (int i = lane; i < hd; i += 32) {
                const float v = x[i] + (b ? b[i] : 0.f);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float inv = w ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.0f;
            T* dst;
            if (head < nh) dst = q_out + ((size_t)n * nh + head) * hd;
            else if (page_id >= 0) dst = k_cache + (((size_t)page_id * nkv + (head - nh)) * page + in_page) * hd;
            else continue;
            const float f = head < nh ? q_factor : 1.0f;
            for (int i = lane; i < hd; i += 32) {
                float v = x[i] + (b ? b[i] : 0.f);
                if (w) v = v * inv * w[i];
                dst[i] = from_f32<T>(v * f);
            }
        } else if (page_id >= 0) {
            const int vh = head - nh - nkv;
            const size_t off = (size_t)(nh + nkv) * hd + (size_t)vh * vd;
            const float* x = src + off;
            const float* b = bias ? bias + off : nullptr;
            T* dst = v_cache + (((size_t)page_id * nkv + vh) * page + in_page) * vd;
            for (int i = lane; i < vd; i += 32) dst[i] = from_f32<T>(x[i] + (b ? b[i] : 0.f));
        }
    }
}

ESP_API int esp_qknorm_kvwrite(const float* qkv, const float* bias, const float* q_w, const float* k_w, float eps,
                               float temp_coef, int temp_every, const int* tok_seq, const int* tok_pos, void* q_out,
                               void* k_cache, void* v_cache, int is_bf16, const int* block_table, int table_stride,
                               int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int vd, int write_kv,
                               int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || vd <= 0 || nkv <= 0 || nh <= 0 || page <= 0) return (int)cudaErrorInvalidValue;
    const int heads = nh + 2 * nkv;
    const int threads = heads >= 8 ? 256 : 32 * heads;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, qknorm_kvwrite_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, qkv, bias, q_w, k_w,
                       eps, temp_coef, temp_every, tok_seq, tok_pos, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, block_table,
                       table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, qknorm_kvwrite_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, qkv, bias, q_w,
                       k_w, eps, temp_coef, temp_every, tok_seq, tok_pos, (float*)q_out, (float*)k_cache, (float*)v_cache,
                       block_table, table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- norms over the whole projection, partial rotation
// qkv: [n_tokens, nh*hd + nkv*hd + nkv*vd] float.  The queries of a token, all heads together, are divided by their
// root mean square over the nh*hd channels (eps inside the root) and multiplied by a weight per channel (q_w, nh*hd
// numbers); the keys likewise over nkv*hd channels with k_w (null: that side is left as projected).  Then the first
// ``rot`` channels of every head are rotated, channel i with channel i + rot/2, by the angle position * inv_freq[i]
// (a 32-bit product; sine and cosine in 32-bit); the other channels pass unchanged.  Values are multiplied by v_scale.
// Queries go to q_out [n_tokens, nh, hd], keys [pages, nkv, PAGE, hd] and values [pages, nkv, PAGE, vd] to the
// token's place in the paged cache.  One block per token.
template <typename T>
__global__ void widenorm_rope_kvwrite_kernel(const float* __restrict__ qkv, const float* __restrict__ q_w,
                                             const float* __restrict__ k_w, float eps, const float* __restrict__ inv_freq,
                                             int rot, float v_scale, const int* __restrict__ tok_seq,
                                             const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_cache,
                                             T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                                             int n_pages, int page, int nh, int nkv, int hd, int vd, int write_kv,
                                             int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int n = blockIdx.x, tid = threadIdx.x;
    const int pos = tok_pos[n], seq = tok_seq[n];
    const int qw = nh * hd, kw = nkv * hd, vw = nkv * vd;
    const float* src = qkv + (size_t)n * (qw + kw + vw);
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (tid == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    float ssq = 0.f, ssk = 0.f;
    for (int e = tid; e < qw; e += blockDim.x) ssq = fmaf(src[e], src[e], ssq);
    for (int e = tid; e < kw; e += blockDim.x) ssk = fmaf(src[qw + e], src[qw + e], ssk);
    const float inv_q = q_w ? 1.0f / sqrtf(block_sum(ssq, scratch) / (float)qw + eps) : 1.0f;
    const float inv_k = k_w ? 1.0f / sqrtf(block_sum(ssk, scratch) / (float)kw + eps) : 1.0f;
    const int half = rot / 2;
    const float p = (float)pos;
    // the row's angles are the same for every head: their cosines and sines are made once (dynamic shared memory:
    // rot floats), from the same expression a head of its own would evaluate
    extern __shared__ float rot_cs[];
    for (int c = tid; c < half; c += blockDim.x) sincosf(p * inv_freq[c], &rot_cs[half + c], &rot_cs[c]);
    __syncthreads();
    for (int e = tid; e < qw + kw; e += blockDim.x) {
        const bool is_q = e < qw;
        const int local = is_q ? e : e - qw;
        const int head = local / hd, c = local - head * hd;
        if (c >= half && c < rot) continue;               // the second half of a pair is written with the first
        const float* w = is_q ? q_w : k_w;
        const float inv = is_q ? inv_q : inv_k;
        T* dst;
        if (is_q) dst = q_out + ((size_t)n * nh + head) * hd;
        else if (page_id >= 0) dst = k_cache + (((size_t)page_id * nkv + head) * page + in_page) * hd;
        else continue;
        float a = src[e];
        if (w) a = a * inv * w[local];
        if (c < half) {
            float b = src[e + half];
            if (w) b = b * inv * w[local + half];
            const float cs = rot_cs[c], sn = rot_cs[half + c];
            dst[c] = from_f32<T>(a * cs - b * sn);
            dst[c + half] = from_f32<T>(b * cs + a * sn);
        } else {
            dst[c] = from_f32<T>(a);
        }
    }
    if (page_id >= 0) {
        for (int e = tid; e < vw; e += blockDim.x) {
            const int head = e / vd, c = e - head * vd;
            v_cache[(((size_t)page_id * nkv + head) * page + in_page) * vd + c] = from_f32<T>(src[qw + kw + e] * v_scale);
        }
    }
}

// The same for head sizes, value sizes and half a rotation of whole pieces of four channels, and aligned buffers.  The
// row's query and key part is read once, in 16-byte loads, into shared memory (the sums of squares are taken on the
// way, both reduced in one exchange).  A thread then makes four
// neighbouring channels and, where they are rotated, their four partners, and stores each as one piece.  Per element the
// arithmetic is that of the kernel above; only the order in which the squares are added differs.
// Dynamic shared memory: (nh * hd + nkv * hd + rot) floats.
template <typename T>
__global__ void __launch_bounds__(256)
widenorm_rope_kvwrite_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ q_w,
                                 const float* __restrict__ k_w, float eps, const float* __restrict__ inv_freq, int rot,
                                 float v_scale, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                 T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                 const int* __restrict__ block_table, int table_stride, int n_pages, int page, int nh,
                                 int nkv, int hd, int vd, int write_kv, int* __restrict__ status) {
    pdl_trigger();
    extern __shared__ __align__(16) float row_smem[];
    __shared__ float part[2][8];
    const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int qw = nh * hd, kw = nkv * hd, vw = nkv * vd, half = rot / 2;
    float* row = row_smem;
    float* rot_cs = row_smem + qw + kw;
    pdl_wait();
    const int pos = tok_pos[n], seq = tok_seq[n];
    const float p = (float)pos;
    for (int c = tid; c < half; c += blockDim.x) sincosf(p * inv_freq[c], &rot_cs[half + c], &rot_cs[c]);
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (tid == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const float* src = qkv + (size_t)n * (qw + kw + vw);
    float ssq = 0.f, ssk = 0.f;
    for (int e = 4 * tid; e < qw + kw; e += 4 * blockDim.x) {
        const float4 v = *reinterpret_cast<const float4*>(src + e);
        *reinterpret_cast<float4*>(row + e) = v;
        const float s4 = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, v.x * v.x)));
        if (e < qw) ssq += s4; else ssk += s4;
    }
    ssq = warp_sum(ssq), ssk = warp_sum(ssk);
    if (lane == 0) part[0][warp] = ssq, part[1][warp] = ssk;
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int i = 0; i < nwarp; i++) tq += part[0][i], tk += part[1][i];
    const float inv_q = q_w ? 1.0f / sqrtf(tq / (float)qw + eps) : 1.0f;
    const float inv_k = k_w ? 1.0f / sqrtf(tk / (float)kw + eps) : 1.0f;
    for (int e = 4 * tid; e < qw + kw; e += 4 * blockDim.x) {
        const bool is_q = e < qw;
        const int local = is_q ? e : e - qw;
        const int head = local / hd, c = local - head * hd;
        if (c >= half && c < rot) continue;               // written with the first halves of their pairs
        const float* w = is_q ? q_w : k_w;
        const float inv = is_q ? inv_q : inv_k;
        T* dst;
        if (is_q) dst = q_out + ((size_t)n * nh + head) * hd;
        else if (page_id >= 0) dst = k_cache + (((size_t)page_id * nkv + head) * page + in_page) * hd;
        else continue;
        const float4 a4 = *reinterpret_cast<const float4*>(row + e);
        float a[4] = {a4.x, a4.y, a4.z, a4.w};
        if (w) {
            const float4 w4 = *reinterpret_cast<const float4*>(w + local);
            a[0] = a[0] * inv * w4.x, a[1] = a[1] * inv * w4.y, a[2] = a[2] * inv * w4.z, a[3] = a[3] * inv * w4.w;
        }
        if (c < half) {
            const float4 b4 = *reinterpret_cast<const float4*>(row + e + half);
            float b[4] = {b4.x, b4.y, b4.z, b4.w};
            if (w) {
                const float4 w4 = *reinterpret_cast<const float4*>(w + local + half);
                b[0] = b[0] * inv * w4.x, b[1] = b[1] * inv * w4.y, b[2] = b[2] * inv * w4.z, b[3] = b[3] * inv * w4.w;
            }
            float lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float cs = rot_cs[c + i], sn = rot_cs[half + c + i];
                lo[i] = a[i] * cs - b[i] * sn;
                hi[i] = b[i] * cs + a[i] * sn;
            }
            Vec4<T>::store(dst + c, lo[0], lo[1], lo[2], lo[3]);
            Vec4<T>::store(dst + c + half, hi[0], hi[1], hi[2], hi[3]);
        } else {
            Vec4<T>::store(dst + c, a[0], a[1], a[2], a[3]);
        }
    }
    if (page_id >= 0) {
        for (int e = 4 * tid; e < vw; e += 4 * blockDim.x) {
            const int head = e / vd, c = e - head * vd;
            const float4 v = *reinterpret_cast<const float4*>(src + qw + kw + e);
            Vec4<T>::store(v_cache + (((size_t)page_id * nkv + head) * page + in_page) * vd + c, v.x * v_scale, v.y * v_scale,
                           v.z * v_scale, v.w * v_scale);
        }
    }
}

ESP_API int esp_widenorm_rope_kvwrite(const float* qkv, const float* q_w, const float* k_w, float eps, const float* inv_freq,
                                      int rot, float v_scale, const int* tok_seq, const int* tok_pos, void* q_out,
                                      void* k_cache, void* v_cache, int is_bf16, const int* block_table, int table_stride,
                                      int n_pages, int page, int n_tokens, int nh, int nkv, int hd, int vd, int write_kv,
                                      int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || vd <= 0 || nkv <= 0 || nh <= 0 || page <= 0 || rot < 0 || rot > hd || rot % 2 != 0 || (rot > 0 && !inv_freq))
        return (int)cudaErrorInvalidValue;
    const int threads = (nh + nkv) * hd >= 2048 ? 256 : 128;
    // which form runs depends on the sizes and the buffers' alignment alone, never on the rows of a step
    const size_t row_bytes = (size_t)((nh + nkv) * hd + rot) * sizeof(float);
    const size_t ptrs = (size_t)qkv | (size_t)q_w | (size_t)k_w | (size_t)q_out | (size_t)k_cache | (size_t)v_cache;
    if (hd % 4 == 0 && vd % 4 == 0 && rot % 8 == 0 && (ptrs & 15) == 0 && row_bytes <= 40 * 1024) {
        if (is_bf16)
            esp_launch_pdl(ESP_PDL_SMALL, widenorm_rope_kvwrite_vec_kernel<bf16>, dim3(n_tokens), dim3(threads), row_bytes, stream,
                           qkv, q_w, k_w, eps, inv_freq, rot, v_scale, tok_seq, tok_pos, (bf16*)q_out, (bf16*)k_cache,
                           (bf16*)v_cache, block_table, table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
        else
            esp_launch_pdl(ESP_PDL_SMALL, widenorm_rope_kvwrite_vec_kernel<float>, dim3(n_tokens), dim3(threads), row_bytes, stream,
                           qkv, q_w, k_w, eps, inv_freq, rot, v_scale, tok_seq, tok_pos, (float*)q_out, (float*)k_cache,
                           (float*)v_cache, block_table, table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
        return esp_launch_status();
    }
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, widenorm_rope_kvwrite_kernel<bf16>, dim3(n_tokens), dim3(threads), rot * sizeof(float), stream, qkv, q_w, k_w,
                       eps, inv_freq, rot, v_scale, tok_seq, tok_pos, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, block_table,
                       table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, widenorm_rope_kvwrite_kernel<float>, dim3(n_tokens), dim3(threads), rot * sizeof(float), stream, qkv, q_w, k_w,
                       eps, inv_freq, rot, v_scale, tok_seq, tok_pos, (float*)q_out, (float*)k_cache, (float*)v_cache,
                       block_table, table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status);
    return esp_launch_status();
}

// ---------------------------------------------------------------- neighbour-pair rotation, unit root mean square per head,
// values blended with those of an earlier layer
// qkv: [n_tokens, nh*hd + nkv*hd + nkv*vd] float, bias (may be null) of the same width.  Of the first ``rot`` channels of
// every query and key head, channel 2i is rotated with channel 2i + 1 by the angle position * inv_freq[i] (a 32-bit
// product; sine and cosine in 32-bit); the other channels pass unchanged.  With ``unit_norm`` every head is then divided
// by its root mean square over hd (eps inside the root; no weight).  Values: blend_mode 1 copies the row's values
// (bias added, unrounded) to v_shared [n_tokens, nkv*vd]; blend_mode 2 replaces them by (1 - lambda) v + lambda v_shared
// with lambda read from the device.  Queries go to q_out [n_tokens, nh, hd], keys [pages, nkv, PAGE, hd] and values
// [pages, nkv, PAGE, vd] to the token's place in the paged cache.  One block per token, a warp a head.
namespace {
constexpr int PAIR_ROPE_MAX_HD = 256;

__device__ __forceinline__ void store_pair(float* dst, float a, float b) { *reinterpret_cast<float2*>(dst) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(bf16* dst, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
}

// PAIRS: head sizes are even and every row starts on an 8-byte boundary, so a lane loads a channel pair as one piece
// and stores it as one; else channel by channel.  Which form runs depends on the sizes and the buffers' alignment alone.
template <typename T, bool PAIRS>
__global__ void pair_rope_unitnorm_kvwrite_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                                  const float* __restrict__ inv_freq, int rot, float eps, int unit_norm,
                                                  float* __restrict__ v_shared, int blend_mode,
                                                  const float* __restrict__ lambda, const int* __restrict__ tok_seq,
                                                  const int* __restrict__ tok_pos, T* __restrict__ q_out,
                                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                  const int* __restrict__ block_table, int table_stride, int n_pages,
                                                  int page, int nh, int nkv, int hd, int vd, int write_kv,
                                                  int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float rope_cs[];                    // [rot / 2] cosines, then [rot / 2] sines of this row's angles
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int pos = tok_pos[n], seq = tok_seq[n];
    const size_t width = (size_t)(nh + nkv) * hd + (size_t)nkv * vd;
    const float* src = qkv + (size_t)n * width;
    int page_id = -1;
    if (write_kv) {
        page_id = block_table[(size_t)seq * table_stride + pos / page];
        if (page_id < 0 || page_id >= n_pages) {
            if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
            page_id = -1;
        }
    }
    const int in_page = pos % page;
    const float p = (float)pos;
    const int half = rot / 2;
    // the row's angles are the same for every head: their cosines and sines are made once
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &rope_cs[half + i], &rope_cs[i]);
    __syncthreads();
    constexpr int PER = PAIR_ROPE_MAX_HD / 64;             // pairs of channels a lane holds
    for (int head = warp; head < nh + 2 * nkv; head += nwarp) {
        if (head < nh + nkv) {
            const float* x = src + (size_t)head * hd;
            const float* b = bias ? bias + (size_t)head * hd : nullptr;
            float lo[PER], hi[PER];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int c = 2 * (lane + 32 * j);
                lo[j] = hi[j] = 0.f;
                if (c >= hd) continue;
                float u, v;
                if (PAIRS) {
                    const float2 xv = *reinterpret_cast<const float2*>(x + c);
                    u = xv.x;
                    v = xv.y;
                    if (b) {
                        const float2 bv = *reinterpret_cast<const float2*>(b + c);
                        u += bv.x;
                        v += bv.y;
                    }
                } else {
                    u = x[c] + (b ? b[c] : 0.f);
                    v = c + 1 < hd ? x[c + 1] + (b ? b[c + 1] : 0.f) : 0.f;
                }
                if (c + 1 < rot) {
                    const float cs = rope_cs[c >> 1], sn = rope_cs[half + (c >> 1)];
                    const float ru = u * cs - v * sn, rv = v * cs + u * sn;
                    u = ru;
                    v = rv;
                }
                lo[j] = u;
                hi[j] = v;
                ss = fmaf(u, u, ss);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            const float inv = unit_norm ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.0f;
            T* dst;
            if (head < nh) dst = q_out + ((size_t)n * nh + head) * hd;
            else if (page_id >= 0) dst = k_cache + (((size_t)page_id * nkv + (head - nh)) * page + in_page) * hd;
            else continue;
#pragma unroll
            for (int j = 0; j < PER; j++) {
                const int c = 2 * (lane + 32 * j);
                if (PAIRS) {
                    if (c < hd) store_pair(dst + c, lo[j] * inv, hi[j] * inv);
                } else {
                    if (c < hd) dst[c] = from_f32<T>(lo[j] * inv);
                    if (c + 1 < hd) dst[c + 1] = from_f32<T>(hi[j] * inv);
                }
            }
        } else {
            const int vh = head - nh - nkv;
            const size_t off = (size_t)(nh + nkv) * hd + (size_t)vh * vd;
            const float* x = src + off;
            const float* b = bias ? bias + off : nullptr;
            float* shared_row = v_shared ? v_shared + (size_t)n * nkv * vd + (size_t)vh * vd : nullptr;
            const float lam = blend_mode == 2 ? lambda[0] : 0.f;
            T* dst = page_id >= 0 ? v_cache + (((size_t)page_id * nkv + vh) * page + in_page) * vd : nullptr;
            if (PAIRS) {
                for (int i = 2 * lane; i < vd; i += 64) {
                    float2 v = *reinterpret_cast<const float2*>(x + i);
                    if (b) {
                        const float2 bv = *reinterpret_cast<const float2*>(b + i);
                        v.x += bv.x;
                        v.y += bv.y;
                    }
                    if (blend_mode == 1) {
                        *reinterpret_cast<float2*>(shared_row + i) = v;
                    } else if (blend_mode == 2) {
                        const float2 f = *reinterpret_cast<const float2*>(shared_row + i);
                        v.x = (1.0f - lam) * v.x + lam * f.x;
                        v.y = (1.0f - lam) * v.y + lam * f.y;
                    }
                    if (dst) store_pair(dst + i, v.x, v.y);
                }
            } else {
                for (int i = lane; i < vd; i += 32) {
                    float v = x[i] + (b ? b[i] : 0.f);
                    if (blend_mode == 1) shared_row[i] = v;
                    else if (blend_mode == 2) v = (1.0f - lam) * v + lam * shared_row[i];
                    if (dst) dst[i] = from_f32<T>(v);
                }
            }
        }
    }
}
}  // namespace

ESP_API int esp_pair_rope_unitnorm_kvwrite(const float* qkv, const float* bias, const float* inv_freq, int rot, float eps,
                                           int unit_norm, float* v_shared, int blend_mode, const float* lambda,
                                           const int* tok_seq, const int* tok_pos, void* q_out, void* k_cache, void* v_cache,
                                           int is_bf16, const int* block_table, int table_stride, int n_pages, int page,
                                           int n_tokens, int nh, int nkv, int hd, int vd, int write_kv, int* status,
                                           cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > PAIR_ROPE_MAX_HD || vd <= 0 || nkv <= 0 || nh <= 0 || page <= 0 || rot < 0 || rot > hd || rot % 2 != 0 ||
        (rot > 0 && !inv_freq) || blend_mode < 0 || blend_mode > 2 || (blend_mode != 0 && !v_shared) ||
        (blend_mode == 2 && !lambda))
        return (int)cudaErrorInvalidValue;
    const int heads = nh + 2 * nkv;
    const int threads = heads >= 8 ? 256 : 32 * heads;
    const size_t smem = (size_t)rot * sizeof(float);
    const size_t ptrs = (size_t)qkv | (size_t)bias | (size_t)v_shared | (size_t)q_out | (size_t)k_cache | (size_t)v_cache;
    const bool pairs = hd % 2 == 0 && vd % 2 == 0 && (ptrs & 7) == 0;
#define ESP_PAIR_ROPE(T, PAIRS)                                                                                              \
    esp_launch_pdl(ESP_PDL_SMALL, pair_rope_unitnorm_kvwrite_kernel<T, PAIRS>, dim3(n_tokens), dim3(threads), smem, stream, qkv,  \
                   bias, inv_freq, rot, eps, unit_norm, v_shared, blend_mode, lambda, tok_seq, tok_pos, (T*)q_out, (T*)k_cache,    \
                   (T*)v_cache, block_table, table_stride, n_pages, page, nh, nkv, hd, vd, write_kv, status)
    if (is_bf16) {
        if (pairs) ESP_PAIR_ROPE(bf16, true);
        else ESP_PAIR_ROPE(bf16, false);
    } else {
        if (pairs) ESP_PAIR_ROPE(float, true);
        else ESP_PAIR_ROPE(float, false);
    }
#undef ESP_PAIR_ROPE
    return esp_launch_status();
}
