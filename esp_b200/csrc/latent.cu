// Attention through a low-rank latent: what is cached per position is one row [latent (rank) | rotated key part
// (rot)], the same for every head.  With the keys' up-projection folded into the queries and the values' up-projection
// applied after the weighted sum, every head attends to the cached rows themselves:
//     score(h, j) = (q_lat[h] . latent_j + q_rot[h] . krot_j) * scale,   q_lat[h] = W_uk[h]^T q_nope[h]
//     o_lat[h]    = sum_j softmax(score)(h, j) latent_j,                 out[h]   = W_uv[h] o_lat[h]
// which is one key/value "head" of width rank + rot (keys) and rank (values, the row's first part) for all
// query heads.  This file holds the cache write (norm of the latent, rotation of the shared key part with
// interpolated frequencies), the rotation of the queries, the per-head products, and the attention over the
// paged rows.  Angles, norms, scores and weights are 32-bit whatever the cache's dtype.
#include "common.cuh"

namespace {

// angle of pair i at position p: p * inv_freq[i]; cos and sin are multiplied by ``mag``
__device__ __forceinline__ void rot_pair(float u, float v, float pos, float f, float mag, float& a, float& b) {
    float s, c;
    sincosf(pos * f, &s, &c);
    s *= mag;
    c *= mag;
    a = u * c - v * s;
    b = v * c + u * s;
}

// ---------------------------------------------------------------------------------------------- cache write
// d: [N, rank + rot] float (the down-projection's output).  Row of the pool: [rank | rot].
template <typename T>
__global__ void latent_kv_store_kernel(const float* __restrict__ d, const float* __restrict__ norm_w,
                                       const float* __restrict__ inv_freq, float mag, int rot_dims,
                                       const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                       const int* __restrict__ block_table, int table_stride, int n_pages, int page,
                                       T* __restrict__ pool, int rank, int rot, float eps, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int n = blockIdx.x, width = rank + rot;
    const float* src = d + (size_t)n * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)rank + eps);
    const int seq = tok_seq[n], pos = tok_pos[n];
    const int pg = block_table[(size_t)seq * table_stride + pos / page];
    if (pg < 0 || pg >= n_pages) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    T* row = pool + ((size_t)pg * page + pos % page) * width;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_f32<T>(src[i] * inv * norm_w[i]);
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
        float o;
        if (i < half) {
            float a, b;
            rot_pair(src[rank + i], src[rank + i + half], (float)pos, inv_freq[i], mag, a, b);
            o = a;
        } else if (i < rot_dims) {
            float a, b;
            rot_pair(src[rank + i - half], src[rank + i], (float)pos, inv_freq[i - half], mag, a, b);
            o = b;
        } else {
            o = src[rank + i];
        }
        row[rank + i] = from_f32<T>(o);
    }
}

// ---------------------------------------------------------------------------------------------- queries
// q: [N, H, nope + rot] float.  The rotated part of every head goes to qx[n, h, rank + :] (qx: [N, H, rank + rot]).
template <typename T>
__global__ void latent_q_rotate_kernel(const float* __restrict__ q, const float* __restrict__ inv_freq, float mag,
                                       int rot_dims, const int* __restrict__ tok_pos, T* __restrict__ qx, int H, int nope,
                                       int rot, int rank) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const float pos = (float)tok_pos[n];
    const int half = rot_dims / 2;
    for (int idx = threadIdx.x; idx < H * rot; idx += blockDim.x) {
        const int h = idx / rot, i = idx - h * rot;
        const float* src = q + ((size_t)n * H + h) * (nope + rot) + nope;
        float o;
        if (i < half) {
            float a, b;
            rot_pair(src[i], src[i + half], pos, inv_freq[i], mag, a, b);
            o = a;
        } else if (i < rot_dims) {
            float a, b;
            rot_pair(src[i - half], src[i], pos, inv_freq[i - half], mag, a, b);
            o = b;
        } else {
            o = src[i];
        }
        qx[((size_t)n * H + h) * (rank + rot) + rank + i] = from_f32<T>(o);
    }
}

// ---------------------------------------------------------------------------------------------- per-head products
// out[n, h, j] = sum_i a[n, h, i] * w[h, j, i]   (i < kin, j < nout); a's and out's heads may be parts of wider rows:
// a[n, h, i] = a[n * lda + h * a_head + i], out[n, h, j] = out[n * ldo + h * o_head + j].
// A block takes ROWS rows of one head; a warp takes output channels in turn, its lanes the input channels, so a
// weight row is read once per ROWS rows; sums run lane-wise in index order and then over a fixed butterfly.
constexpr int PH_ROWS = 8;
constexpr int PH_OUTS = 16;       // output channels of a block
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(128)
per_head_linear_kernel(const TA* __restrict__ a, long long lda, int a_head, const TW* __restrict__ w, TO* __restrict__ out,
                       long long ldo, int o_head, int n_rows, int kin, int nout) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float as[];                  // [PH_ROWS][kin]
    const int n0 = blockIdx.x * PH_ROWS, h = blockIdx.y;
    const int rows = min(PH_ROWS, n_rows - n0);
    for (int idx = threadIdx.x; idx < PH_ROWS * kin; idx += blockDim.x) {
        const int r = idx / kin, i = idx - r * kin;
        as[idx] = r < rows ? to_f32(a[(size_t)(n0 + r) * lda + (size_t)h * a_head + i]) : 0.f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TW* wh = w + (size_t)h * nout * kin;
    const int j_end = min(nout, ((int)blockIdx.z + 1) * PH_OUTS);
    for (int j = blockIdx.z * PH_OUTS + warp; j < j_end; j += 4) {
        float acc[PH_ROWS];
#pragma unroll
        for (int r = 0; r < PH_ROWS; r++) acc[r] = 0.f;
        for (int i = lane; i < kin; i += 32) {
            const float wv = to_f32(wh[(size_t)j * kin + i]);
#pragma unroll
            for (int r = 0; r < PH_ROWS; r++) acc[r] = fmaf(as[r * kin + i], wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < PH_ROWS; r++) {
            if (r >= rows) break;                   // the same for every lane
            const float s = warp_sum(acc[r]);
            if (lane == 0) out[(size_t)(n0 + r) * ldo + (size_t)h * o_head + j] = from_f32<TO>(s);
        }
    }
}

// The same product on the tensor cores for many rows and bfloat16 weights: a block takes 64 rows x 64 output channels
// of one head, four warps 32 x 32 each, the input channels in pieces of 32 through shared memory (inputs are rounded
// to bfloat16 as they are staged; sums are float).
constexpr int PHM_MIN_ROWS = 17;
constexpr int PHM_T = 64, PHM_KC = 32, PHM_LD = PHM_KC + 8;

__device__ __forceinline__ void phm_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void phm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load8(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 load8(const float* p) {
    const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
    __nv_bfloat162 a = __floats2bfloat162_rn(lo.x, lo.y), b = __floats2bfloat162_rn(lo.z, lo.w);
    __nv_bfloat162 c = __floats2bfloat162_rn(hi.x, hi.y), d = __floats2bfloat162_rn(hi.z, hi.w);
    return make_uint4(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b), *reinterpret_cast<unsigned*>(&c),
                      *reinterpret_cast<unsigned*>(&d));
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(128)
per_head_mma_kernel(const TA* __restrict__ a, long long lda, int a_head, const bf16* __restrict__ w, TO* __restrict__ out,
                    long long ldo, int o_head, int n_rows, int kin, int nout) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) bf16 as[PHM_T * PHM_LD];
    __shared__ __align__(16) bf16 ws[PHM_T * PHM_LD];
    const int n0 = blockIdx.x * PHM_T, h = blockIdx.y, j0 = blockIdx.z * PHM_T;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int wr = (warp & 1) * 32, wc = (warp >> 1) * 32;
    const bf16* wh = w + (size_t)h * nout * kin;
    // every piece of eight channels starts on a 16-byte boundary (32 for float inputs)
    const bool wide = kin % 8 == 0 && lda % 8 == 0 && a_head % 8 == 0 && ((size_t)a % 32) == 0 && ((size_t)w % 16) == 0;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[i][j][k] = 0.f;
    for (int k0 = 0; k0 < kin; k0 += PHM_KC) {
        __syncthreads();
        if (wide) {
            // eight channels a piece: 16 bytes of bfloat16, or two float4 rounded to bfloat16 on the way
            for (int idx = tid; idx < PHM_T * (PHM_KC / 8); idx += 128) {
                const int r = idx / (PHM_KC / 8), c = (idx - r * (PHM_KC / 8)) * 8;
                const int k = k0 + c;
                uint4 av = make_uint4(0u, 0u, 0u, 0u), wv = make_uint4(0u, 0u, 0u, 0u);
                if (k < kin && n0 + r < n_rows) av = load8(a + (size_t)(n0 + r) * lda + (size_t)h * a_head + k);
                if (k < kin && j0 + r < nout) wv = *reinterpret_cast<const uint4*>(wh + (size_t)(j0 + r) * kin + k);
                *reinterpret_cast<uint4*>(as + r * PHM_LD + c) = av;
                *reinterpret_cast<uint4*>(ws + r * PHM_LD + c) = wv;
            }
        } else {
            for (int idx = tid; idx < PHM_T * PHM_KC; idx += 128) {
                const int r = idx / PHM_KC, c = idx - r * PHM_KC;
                const int k = k0 + c;
                const bool kin_ok = k < kin;
                as[r * PHM_LD + c] = (kin_ok && n0 + r < n_rows)
                    ? __float2bfloat16_rn(to_f32(a[(size_t)(n0 + r) * lda + (size_t)h * a_head + k])) : __float2bfloat16_rn(0.f);
                ws[r * PHM_LD + c] = (kin_ok && j0 + r < nout) ? wh[(size_t)(j0 + r) * kin + k] : __float2bfloat16_rn(0.f);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < PHM_KC / 16; kk++) {
            unsigned af[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
                phm_ldmatrix_x4(af[mt], as + (wr + mt * 16 + (lane & 15)) * PHM_LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                unsigned bfr[4];
                phm_ldmatrix_x4(bfr, ws + (wc + nb * 16 + (lane & 7) + (lane >> 4) * 8) * PHM_LD + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    phm_mma(acc[mt][2 * nb], af[mt], bfr[0], bfr[1]);
                    phm_mma(acc[mt][2 * nb + 1], af[mt], bfr[2], bfr[3]);
                }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = n0 + wr + mt * 16 + g + 8 * (e >> 1), j = j0 + wc + nt * 8 + tg * 2 + (e & 1);
                if (r < n_rows && j < nout) out[(size_t)r * ldo + (size_t)h * o_head + j] = from_f32<TO>(acc[mt][nt][e]);
            }
}

int launch_per_head_mma(const void* a, int a_dtype, long long lda, int a_head, const void* w, void* out, int o_dtype,
                        long long ldo, int o_head, int n_rows, int H, int kin, int nout, cudaStream_t stream) {
    dim3 grid((n_rows + PHM_T - 1) / PHM_T, H, (nout + PHM_T - 1) / PHM_T);
#define ESP_PHM(TA, TO)                                                                                                     \
    esp_launch_pdl(0, per_head_mma_kernel<TA, TO>, grid, dim3(128), 0, stream, (const TA*)a, lda, a_head,                     \
                   (const bf16*)w, (TO*)out, ldo, o_head, n_rows, kin, nout)
    switch (a_dtype * 2 + o_dtype) {
        case 0: ESP_PHM(float, float); break;
        case 1: ESP_PHM(float, bf16); break;
        case 2: ESP_PHM(bf16, float); break;
        default: ESP_PHM(bf16, bf16); break;
    }
#undef ESP_PHM
    return esp_launch_status();
}

// ---------------------------------------------------------------------------------------------- attention
// One block per (token, group of heads): the cached rows of a chunk of 32 positions are staged once in shared
// memory (as float) and used by every head of the group.  A warp owns HW heads; for a head, lane j scores key j of
// the chunk, the running maximum and sum are kept per head, and lane l accumulates the value channels l, l + 32, ...
// Chunks are aligned to absolute multiples of 32, so the order of every addition depends on the query's position
// and the window alone.
constexpr int LA_CHUNK = 32;
constexpr int LA_WARPS = 4;

template <typename T, int VR, int HW>
__global__ void __launch_bounds__(LA_WARPS * 32)
attn_latent_kernel(const T* __restrict__ qx, const T* __restrict__ pool, T* __restrict__ out,
                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ block_table,
                   int table_stride, int n_pages, int page, int H, int hdk, int hdv, int window, float scale,
                   int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int stride = hdk + 1;                    // rows of the chunk one bank apart
    float* rows = sm;                              // [LA_CHUNK][stride]
    float* qs = sm + LA_CHUNK * stride;            // [LA_WARPS * HW][hdk]
    __shared__ int pages[LA_CHUNK];
    const int n = blockIdx.x, h0 = blockIdx.y * (LA_WARPS * HW);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = tok_seq[n], pos = tok_pos[n];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int idx = tid; idx < LA_WARPS * HW * hdk; idx += blockDim.x) {
        const int hh = idx / hdk, i = idx - hh * hdk;
        const int h = h0 + hh;
        qs[idx] = h < H ? to_f32(qx[((size_t)n * H + h) * hdk + i]) : 0.f;
    }
    float m_run[HW], l_run[HW], acc[HW][VR];
#pragma unroll
    for (int a = 0; a < HW; a++) {
        m_run[a] = -INFINITY;
        l_run[a] = 0.f;
#pragma unroll
        for (int i = 0; i < VR; i++) acc[a][i] = 0.f;
    }
    for (int c = lo / LA_CHUNK; c <= pos / LA_CHUNK; c++) {
        const int j0 = c * LA_CHUNK;
        __syncthreads();                           // the chunk before is no longer read (and qs is written)
        if (tid < LA_CHUNK) {
            const int j = j0 + tid;
            int pg = -1;
            if (j >= lo && j <= pos) {
                pg = block_table[(size_t)seq * table_stride + j / page];
                if (pg < 0 || pg >= n_pages) {
                    atomicOr(status, ESP_STATUS_BAD_INDEX);
                    pg = -1;
                }
            }
            pages[tid] = pg;
        }
        __syncthreads();
        for (int idx = tid; idx < LA_CHUNK * hdk; idx += blockDim.x) {
            const int t = idx / hdk, i = idx - t * hdk;
            const int pg = pages[t];
            rows[t * stride + i] = pg >= 0 ? to_f32(pool[((size_t)pg * page + (j0 + t) % page) * hdk + i]) : 0.f;
        }
        __syncthreads();
        const bool seen = pages[lane] >= 0;
#pragma unroll
        for (int a = 0; a < HW; a++) {
            const int hh = warp * HW + a;
            if (h0 + hh >= H) continue;
            const float* qh = qs + hh * hdk;
            const float* kr = rows + lane * stride;
            float dot = 0.f;
            for (int i = 0; i < hdk; i++) dot = fmaf(qh[i], kr[i], dot);
            const float s = seen ? dot * scale : -INFINITY;
            const float m_new = fmaxf(m_run[a], warp_max(s));
            if (m_new == -INFINITY) continue;
            const float p = seen ? expf(s - m_new) : 0.f;
            const float rescale = expf(m_run[a] - m_new);
            l_run[a] = l_run[a] * rescale + warp_sum(p);
            m_run[a] = m_new;
#pragma unroll
            for (int i = 0; i < VR; i++) acc[a][i] *= rescale;
            for (int t = 0; t < LA_CHUNK; t++) {
                const float pt = __shfl_sync(0xffffffffu, p, t);
                if (pt == 0.f) continue;
                const float* vr = rows + t * stride;
#pragma unroll
                for (int i = 0; i < VR; i++) {
                    const int dch = lane + 32 * i;
                    if (dch < hdv) acc[a][i] = fmaf(pt, vr[dch], acc[a][i]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < HW; a++) {
        const int h = h0 + warp * HW + a;
        if (h >= H) continue;
#pragma unroll
        for (int i = 0; i < VR; i++) {
            const int dch = lane + 32 * i;
            if (dch < hdv) out[((size_t)n * H + h) * hdv + dch] = from_f32<T>(l_run[a] > 0.f ? acc[a][i] / l_run[a] : 0.f);
        }
    }
}

template <typename T, int VR, int HW>
int launch_attn_latent(const void* qx, const void* pool, void* out, const int* tok_seq, const int* tok_pos,
                       const int* block_table, int table_stride, int n_pages, int page, int n_tokens, int H, int hdk, int hdv,
                       int window, float scale, int* status, cudaStream_t stream) {
    const size_t smem = ((size_t)LA_CHUNK * (hdk + 1) + (size_t)LA_WARPS * HW * hdk) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = attn_latent_kernel<T, VR, HW>;
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set = true; }
    dim3 grid(n_tokens, (H + LA_WARPS * HW - 1) / (LA_WARPS * HW));
    esp_launch_pdl(ESP_PDL_ATTENTION, kernel, grid, dim3(LA_WARPS * 32), smem, stream, (const T*)qx, (const T*)pool, (T*)out,
                   tok_seq, tok_pos, block_table, table_stride, n_pages, page, H, hdk, hdv, window, scale, status);
    return esp_launch_status();
}

template <typename T, int VR>
int pick_hw(int H, const void* qx, const void* pool, void* out, const int* tok_seq, const int* tok_pos, const int* block_table,
            int table_stride, int n_pages, int page, int n_tokens, int hdk, int hdv, int window, float scale, int* status,
            cudaStream_t stream) {
    constexpr int HW_MAX = VR >= 16 ? 2 : 4;
    const int per_warp = (H + LA_WARPS - 1) / LA_WARPS;
#define ESP_LA(HW_) return launch_attn_latent<T, VR, HW_>(qx, pool, out, tok_seq, tok_pos, block_table, table_stride, n_pages, \
                                                         page, n_tokens, H, hdk, hdv, window, scale, status, stream)
    if (per_warp >= 4 && HW_MAX >= 4) ESP_LA(4);
    if (per_warp >= 2) ESP_LA(2);
    ESP_LA(1);
#undef ESP_LA
}

template <typename T>
int pick_vr(int H, const void* qx, const void* pool, void* out, const int* tok_seq, const int* tok_pos, const int* block_table,
            int table_stride, int n_pages, int page, int n_tokens, int hdk, int hdv, int window, float scale, int* status,
            cudaStream_t stream) {
#define ESP_LA(VR_) return pick_hw<T, VR_>(H, qx, pool, out, tok_seq, tok_pos, block_table, table_stride, n_pages, page, \
                                          n_tokens, hdk, hdv, window, scale, status, stream)
    if (hdv <= 64) ESP_LA(2);
    if (hdv <= 128) ESP_LA(4);
    if (hdv <= 256) ESP_LA(8);
    ESP_LA(16);
#undef ESP_LA
}
// y[n, h, :] = o[n, h, :] * sigmoid(gate[n * ldg + h]): one number per token and head on the head's whole output.
// VEC: head sizes of whole pieces of four channels on aligned buffers: a thread takes a piece.
__device__ __forceinline__ float4 gate_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 gate_load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}
template <typename TI, typename T, bool VEC>
__global__ void head_scalar_gate_kernel(const TI* __restrict__ o, const float* __restrict__ gate, long long ldg,
                                        T* __restrict__ y, long long total, int H, int V) {
    pdl_trigger();
    pdl_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const long long pieces = total / 4;
        const int per_head = V / 4;
        for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < pieces; q += step) {
            const long long nh = q / per_head;
            const long long n = nh / H;
            const int h = (int)(nh - n * H);
            const float s = 1.0f / (1.0f + expf(-gate[n * ldg + h]));
            const float4 v = gate_load4(o + 4 * q);
            Vec4<T>::store(y + 4 * q, v.x * s, v.y * s, v.z * s, v.w * s);
        }
        return;
    }
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += step) {
        const long long nh = idx / V;
        const long long n = nh / H;
        const int h = (int)(nh - n * H);
        const float g = gate[n * ldg + h];
        y[idx] = from_f32<T>(to_f32(o[idx]) * (1.0f / (1.0f + expf(-g))));
    }
}

// Keys and values of every head of the step's tokens, made from their latents, into pages of their own: k float
// [rows, H * K] and v float [rows, H * V] (with their row strides) go to k_pool [pages, H, page, K] and v_pool
// [pages, H, page, V] at the token's place, the page of position p of sequence s being table[s * stride + p / page].
// K and V are multiples of four.  One block a token.
template <typename T>
__global__ void heads_to_pages_kernel(const float* __restrict__ k, long long ldk, const float* __restrict__ v, long long ldv,
                                      const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                      const int* __restrict__ table, int table_stride, int n_pages, int page,
                                      T* __restrict__ k_pool, T* __restrict__ v_pool, int H, int K, int V,
                                      int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int seq = tok_seq[n], pos = tok_pos[n];
    const int pg = table[(size_t)seq * table_stride + pos / page];
    if (pg < 0 || pg >= n_pages) {
        if (threadIdx.x == 0) atomicOr(status, ESP_STATUS_BAD_INDEX);
        return;
    }
    const int in_page = pos % page;
    for (int e = threadIdx.x * 4; e < H * K; e += blockDim.x * 4) {
        const int head = e / K, c = e - head * K;
        const float4 x = *reinterpret_cast<const float4*>(k + (size_t)n * ldk + e);
        Vec4<T>::store(k_pool + (((size_t)pg * H + head) * page + in_page) * K + c, x.x, x.y, x.z, x.w);
    }
    for (int e = threadIdx.x * 4; e < H * V; e += blockDim.x * 4) {
        const int head = e / V, c = e - head * V;
        const float4 x = *reinterpret_cast<const float4*>(v + (size_t)n * ldv + e);
        Vec4<T>::store(v_pool + (((size_t)pg * H + head) * page + in_page) * V + c, x.x, x.y, x.z, x.w);
    }
}
}  // namespace

ESP_API int esp_latent_kv_store(const float* d, const float* norm_w, const float* inv_freq, float mag, int rot_dims,
                                const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride, int n_pages,
                                int page, void* pool, int pool_is_bf16, int n_tokens, int rank, int rot, float eps, int* status,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dims % 2 != 0 || rot_dims > rot || rank <= 0) return (int)cudaErrorInvalidValue;
    const int threads = rank >= 512 ? 256 : 128;
    if (pool_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, latent_kv_store_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, d, norm_w, inv_freq,
                       mag, rot_dims, tok_seq, tok_pos, block_table, table_stride, n_pages, page, (bf16*)pool, rank, rot, eps,
                       status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, latent_kv_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, d, norm_w,
                       inv_freq, mag, rot_dims, tok_seq, tok_pos, block_table, table_stride, n_pages, page, (float*)pool, rank,
                       rot, eps, status);
    return esp_launch_status();
}

ESP_API int esp_latent_q_rotate(const float* q, const float* inv_freq, float mag, int rot_dims, const int* tok_pos, void* qx,
                                int qx_is_bf16, int n_tokens, int H, int nope, int rot, int rank, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dims % 2 != 0 || rot_dims > rot) return (int)cudaErrorInvalidValue;
    if (qx_is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, latent_q_rotate_kernel<bf16>, dim3(n_tokens), dim3(128), 0, stream, q, inv_freq, mag,
                       rot_dims, tok_pos, (bf16*)qx, H, nope, rot, rank);
    else
        esp_launch_pdl(ESP_PDL_SMALL, latent_q_rotate_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, q, inv_freq, mag,
                       rot_dims, tok_pos, (float*)qx, H, nope, rot, rank);
    return esp_launch_status();
}

// dtype codes: 0 = float, 1 = bfloat16
ESP_API int esp_per_head_linear(const void* a, int a_dtype, long long lda, int a_head, const void* w, int w_dtype, void* out,
                                int o_dtype, long long ldo, int o_head, int n_rows, int H, int kin, int nout,
                                cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H > 65535 || (size_t)PH_ROWS * kin * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (w_dtype == 1 && n_rows >= PHM_MIN_ROWS)
        return launch_per_head_mma(a, a_dtype, lda, a_head, w, out, o_dtype, ldo, o_head, n_rows, H, kin, nout, stream);
    dim3 grid((n_rows + PH_ROWS - 1) / PH_ROWS, H, (nout + PH_OUTS - 1) / PH_OUTS);
    const size_t smem = (size_t)PH_ROWS * kin * sizeof(float);
#define ESP_CASE(code_, TA, TW, TO)                                                                                          \
    case code_:                                                                                                             \
        esp_launch_pdl(ESP_PDL_SMALL, per_head_linear_kernel<TA, TW, TO>, grid, dim3(128), smem, stream, (const TA*)a, lda,   \
                       a_head, (const TW*)w, (TO*)out, ldo, o_head, n_rows, kin, nout);                                      \
        break;
    switch (a_dtype * 4 + w_dtype * 2 + o_dtype) {
        ESP_CASE(0, float, float, float)
        ESP_CASE(1, float, float, bf16)
        ESP_CASE(2, float, bf16, float)
        ESP_CASE(3, float, bf16, bf16)
        ESP_CASE(4, bf16, float, float)
        ESP_CASE(5, bf16, float, bf16)
        ESP_CASE(6, bf16, bf16, float)
        ESP_CASE(7, bf16, bf16, bf16)
        default: return (int)cudaErrorInvalidValue;
    }
#undef ESP_CASE
    return esp_launch_status();
}

// qx: [N, H, hdk]; pool: [pages, page, hdk]; out: [N, H, hdv]; values are the first hdv channels of a row.
ESP_API int esp_attn_latent(const void* qx, const void* pool, void* out, int is_bf16, const int* tok_seq, const int* tok_pos,
                            const int* block_table, int table_stride, int n_pages, int page, int n_tokens, int H, int hdk,
                            int hdv, int window, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hdv > hdk || hdv > 512 || hdv <= 0 || H <= 0) return (int)cudaErrorInvalidValue;
    if (is_bf16)
        return pick_vr<bf16>(H, qx, pool, out, tok_seq, tok_pos, block_table, table_stride, n_pages, page, n_tokens, hdk, hdv,
                             window, scale, status, stream);
    return pick_vr<float>(H, qx, pool, out, tok_seq, tok_pos, block_table, table_stride, n_pages, page, n_tokens, hdk, hdv,
                          window, scale, status, stream);
}

ESP_API int esp_head_scalar_gate(const void* o, int o_is_bf16, const float* gate, long long ldg, void* y, int y_is_bf16,
                                 int n_rows, int H, int V, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || V <= 0) return (int)cudaErrorInvalidValue;
    const long long total = (long long)n_rows * H * V;
    const bool vec = V % 4 == 0 && (((size_t)o | (size_t)y) & 15) == 0;      // from sizes and alignment alone
    const long long items = vec ? total / 4 : total;
    const int blocks = (int)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
#define ESP_HEAD_GATE(TI, T, VEC)                                                                                         \
    esp_launch_pdl(ESP_PDL_SMALL, head_scalar_gate_kernel<TI, T, VEC>, dim3(blocks), dim3(256), 0, stream, (const TI*)o, gate, \
                   ldg, (T*)y, total, H, V)
#define ESP_HEAD_GATE_T(TI, T)                                                                                            \
    do {                                                                                                                  \
        if (vec) ESP_HEAD_GATE(TI, T, true);                                                                              \
        else ESP_HEAD_GATE(TI, T, false);                                                                                 \
    } while (0)
    if (o_is_bf16 && y_is_bf16) ESP_HEAD_GATE_T(bf16, bf16);
    else if (o_is_bf16) ESP_HEAD_GATE_T(bf16, float);
    else if (y_is_bf16) ESP_HEAD_GATE_T(float, bf16);
    else ESP_HEAD_GATE_T(float, float);
#undef ESP_HEAD_GATE_T
#undef ESP_HEAD_GATE
    return esp_launch_status();
}

ESP_API int esp_heads_to_pages(const float* k, long long ldk, const float* v, long long ldv, const int* tok_seq,
                               const int* tok_pos, const int* table, int table_stride, int n_pages, int page, void* k_pool,
                               void* v_pool, int is_bf16, int n_rows, int H, int K, int V, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || K <= 0 || V <= 0 || K % 4 != 0 || V % 4 != 0 || ldk % 4 != 0 || ldv % 4 != 0 || page <= 0 ||
        (((size_t)k | (size_t)v | (size_t)k_pool | (size_t)v_pool) & 15) != 0)
        return (int)cudaErrorInvalidValue;
    if (is_bf16)
        esp_launch_pdl(ESP_PDL_SMALL, heads_to_pages_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, k, ldk, v, ldv, tok_seq,
                       tok_pos, table, table_stride, n_pages, page, (bf16*)k_pool, (bf16*)v_pool, H, K, V, status);
    else
        esp_launch_pdl(ESP_PDL_SMALL, heads_to_pages_kernel<float>, dim3(n_rows), dim3(256), 0, stream, k, ldk, v, ldv, tok_seq,
                       tok_pos, table, table_stride, n_pages, page, (float*)k_pool, (float*)v_pool, H, K, V, status);
    return esp_launch_status();
}
