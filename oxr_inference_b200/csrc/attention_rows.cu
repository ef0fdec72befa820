// Paged attention with the sizes and the mask as arguments, one warp per (query token, query head), all in fp32:
//
//   * key size DK and value size DV differ freely; values may be the first DV entries of the key rows (a latent cache:
//     one shared row per token that is both key and value);
//   * mask: causal, optionally within chunks counted from position 0 (i sees j <= i with floor(i/chunk) == floor(j/chunk))
//     or within a window (the last `window` keys), beside which the first `keep_first` keys of the sequence stay visible;
//   * an additive bias by distance, read from a table [distances, heads] (the last row stands for every larger distance);
//   * a sink: a per-head number that joins the softmax denominator as exp(sink) and has no value.
//
// Scores, weights and sums are fp32; T is the type of q, of the cache and of the output. A row's result depends only on
// its position and the keys it sees: keys are taken 32 at a time from the first visible one, whatever the step holds.
// This is the engine's 32-bit attention for these masks and the reference form of its 16-bit one.
//
// Also here: the cache writers of these mixers (rows scattered to slots; the latent row = RMSNorm of the compressed part
// beside the rotated shared key part, with the queries' rotated parts turned in place) and a per-head linear map.
#include "common.cuh"

constexpr int ROWS_MAX_DV_CHUNKS = 32;   // DV <= 1024

// DVC: 32-wide pieces of a value row that a lane accumulates (DV <= 32 * DVC).
template <typename T, int DVC>
__global__ void __launch_bounds__(128) attn_rows_kernel(
    T* __restrict__ out, const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, long long k_slot_stride, int k_head_stride,
    const T* __restrict__ v_pool, long long v_slot_stride, int v_head_stride, int DK, int DV, int H, int KVH, const int* __restrict__ positions,
    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_width, int page_size, int num_pages, float scale,
    int chunk, int window, int keep_first, const float* __restrict__ dist_bias, int bias_rows, const float* __restrict__ sink, int* status) {
    extern __shared__ float q_smem[];   // [warps, DK]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * warps + warp;
    if (h >= H) return;
    const int kvh = h / (H / KVH), r = req_of_token[t], p = positions[t];
    float* qs = q_smem + warp * DK;
    for (int d = lane; d < DK; d += 32) qs[d] = Num<T>::to_f32(q[(size_t)t * q_stride + h * DK + d]) * scale;
    __syncwarp();

    int lo = 0;
    if (chunk > 0) lo = p / chunk * chunk;
    if (window > 0 && p - window + 1 > lo) lo = p - window + 1;
    const int* table = block_table + (size_t)r * table_width;

    float m = -INFINITY, l = 0.f;
    if (sink != nullptr) { m = sink[h]; l = 1.f; }   // a key with score sink[h] and no value
    float acc[DVC];
#pragma unroll
    for (int i = 0; i < DVC; ++i) acc[i] = 0.f;

    // two stretches of keys: the sequence's first keys that stay visible behind the window (none without one), then the window
    const int kept_end = min(keep_first, lo);
    for (int j0 = kept_end > 0 ? 0 : lo; j0 <= p; j0 = (j0 < lo && j0 + 32 >= kept_end) ? lo : j0 + 32) {
        const int last = j0 < lo ? kept_end - 1 : p;      // last key of this stretch
        const int j = j0 + lane;
        const bool seen = j <= last;
        long long slot = 0;
        float s = -INFINITY;
        if (seen) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                oxr_report(status, OXR_BAD_PAGE, t);
            } else {
                slot = (long long)page * page_size + j % page_size;
                const T* kr = k_pool + slot * k_slot_stride + (long long)kvh * k_head_stride;
                float dot = 0.f;
                for (int d = 0; d < DK; ++d) dot = fmaf(qs[d], Num<T>::to_f32(kr[d]), dot);
                s = dot;
                if (dist_bias != nullptr) {
                    const int n = p - j;
                    s += dist_bias[(size_t)(n < bias_rows ? n : bias_rows - 1) * H + h];
                }
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = expf(m - m_new);          // m = -inf: 0
        const float w = seen ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(w);
        m = m_new;
#pragma unroll
        for (int i = 0; i < DVC; ++i) acc[i] *= corr;
        const int count = min(32, last - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float wj = __shfl_sync(0xffffffffu, w, jj);
            const long long sj = __shfl_sync(0xffffffffu, slot, jj);
            const T* vr = v_pool + sj * v_slot_stride + (long long)kvh * v_head_stride;
#pragma unroll
            for (int i = 0; i < DVC; ++i) {
                const int d = lane + 32 * i;
                if (d < DV) acc[i] = fmaf(wj, Num<T>::to_f32(vr[d]), acc[i]);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + ((size_t)t * H + h) * DV;
#pragma unroll
    for (int i = 0; i < DVC; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) o[d] = Num<T>::from_f32(acc[i] * inv);
    }
}

OXR_API int oxr_attention_rows(void* out, const void* q, int q_stride, const void* k_pool, long long k_slot_stride, int k_head_stride,
                               const void* v_pool, long long v_slot_stride, int v_head_stride, int DK, int DV, int H, int KVH, int n_tokens,
                               const int* positions, const int* req_of_token, const int* block_table, int table_width, int page_size, int num_pages,
                               float scale, int chunk, int window, int keep_first, const float* dist_bias, int bias_rows, const float* sink, int dtype,
                               int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (DK <= 0 || DV <= 0 || DV > 32 * ROWS_MAX_DV_CHUNKS || H <= 0 || KVH <= 0 || H % KVH || page_size <= 0 || chunk < 0 || window < 0 || keep_first < 0 ||
        (dist_bias != nullptr && bias_rows <= 0))
        return OXR_BAD_ARGUMENT;
    const int warps = H >= 4 ? 4 : H;
    dim3 grid(n_tokens, (H + warps - 1) / warps);
    if (grid.y > 65535) return OXR_BAD_ARGUMENT;
    const size_t smem = (size_t)warps * DK * sizeof(float);
    if (smem > 48 * 1024) return OXR_BAD_ARGUMENT;
#define OXR_ROWS(T, DVC) \
    attn_rows_kernel<T, DVC><<<grid, 32 * warps, smem, stream>>>((T*)out, (const T*)q, q_stride, (const T*)k_pool, k_slot_stride, k_head_stride, \
                                                                (const T*)v_pool, v_slot_stride, v_head_stride, DK, DV, H, KVH, positions, req_of_token, \
                                                                block_table, table_width, page_size, num_pages, scale, chunk, window, keep_first, dist_bias, \
                                                                bias_rows, sink, status)
    if (dtype == 0) {
        if (DV <= 128) OXR_ROWS(float, 4);
        else if (DV <= 512) OXR_ROWS(float, 16);
        else OXR_ROWS(float, 32);
    } else {
        if (DV <= 128) OXR_ROWS(__nv_bfloat16, 4);
        else if (DV <= 512) OXR_ROWS(__nv_bfloat16, 16);
        else OXR_ROWS(__nv_bfloat16, 32);
    }
#undef OXR_ROWS
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- cache writers
// pool[slots[t], 0:width] = src[t, col0 : col0 + width]; a slot of -1 skips the row. With a second pool (keys and values of one
// token): pool2[slots[t], 0:width2] = src[t, col0 + width : col0 + width + width2] in the same launch.
template <typename T>
__global__ void scatter_rows_kernel(T* __restrict__ pool, long long slot_stride, long long pool_slots, const T* __restrict__ src, int src_stride, int col0,
                                    int width, const int* __restrict__ slots, int* status, T* __restrict__ pool2, long long slot_stride2, int width2) {
    const int t = blockIdx.x;
    const int slot = slots[t];
    if (slot < 0) return;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) oxr_report(status, OXR_BAD_SLOT, t);
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) pool[(long long)slot * slot_stride + i] = src[(size_t)t * src_stride + col0 + i];
    if (pool2 != nullptr)
        for (int i = threadIdx.x; i < width2; i += blockDim.x) pool2[(long long)slot * slot_stride2 + i] = src[(size_t)t * src_stride + col0 + width + i];
}

OXR_API int oxr_scatter_rows(void* pool, long long slot_stride, long long pool_slots, const void* src, int src_stride, int col0, int width,
                             const int* slots, int n_tokens, int dtype, int* status, void* pool2, long long slot_stride2, int width2,
                             cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return 0;
    if (dtype == 0)
        scatter_rows_kernel<float><<<n_tokens, 128, 0, stream>>>((float*)pool, slot_stride, pool_slots, (const float*)src, src_stride, col0, width, slots, status,
                                                                (float*)pool2, slot_stride2, width2);
    else
        scatter_rows_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>((__nv_bfloat16*)pool, slot_stride, pool_slots, (const __nv_bfloat16*)src, src_stride, col0,
                                                                        width, slots, status, (__nv_bfloat16*)pool2, slot_stride2, width2);
    return oxr_launch_status();
}

// One block per token. down[t] = [rank compressed | rot shared key part]:
//   pool[slot] = [ rmsnorm(compressed) * weight | rotate(key part) ]        (skipped for slot -1)
//   q_out[t, h, qo_rot0 : qo_rot0 + rot] = rotate(q[t, h, q_rot0 : q_rot0 + rot])  for every head (q_out may be q)
// rotate: entries 2i and 2i+1 of the first 2 * half entries turn by the token's angle i; the rest pass unchanged.
template <typename T>
__global__ void latent_prep_kernel(T* __restrict__ pool, long long slot_stride, long long pool_slots, const T* __restrict__ down, int rank, int rot,
                                   const float* __restrict__ weight, float eps, const T* q, int heads, int q_head_dim, int q_rot0, T* q_out,
                                   int qo_head_dim, int qo_rot0, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half, const int* __restrict__ slots, int* status) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const T* row = down + (size_t)t * (rank + rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = Num<T>::to_f32(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    const float* c = cos_t + (size_t)t * half;
    const float* s = sin_t + (size_t)t * half;
    const int slot = slots[t];
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) oxr_report(status, OXR_BAD_SLOT, t);
    } else if (slot >= 0) {
        T* dst = pool + (long long)slot * slot_stride;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = Num<T>::from_f32(Num<T>::to_f32(row[i]) * inv * weight[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = Num<T>::to_f32(row[rank + 2 * i]), v = Num<T>::to_f32(row[rank + 2 * i + 1]);
            dst[rank + 2 * i] = Num<T>::from_f32(u * c[i] - v * s[i]);
            dst[rank + 2 * i + 1] = Num<T>::from_f32(v * c[i] + u * s[i]);
        }
        for (int i = 2 * half + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = row[rank + i];
    }
    for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
        const int h = i / half, k = i % half;
        const T* qr = q + ((size_t)t * heads + h) * q_head_dim + q_rot0;
        T* qo = q_out + ((size_t)t * heads + h) * qo_head_dim + qo_rot0;
        const float u = Num<T>::to_f32(qr[2 * k]), v = Num<T>::to_f32(qr[2 * k + 1]);
        qo[2 * k] = Num<T>::from_f32(u * c[k] - v * s[k]);
        qo[2 * k + 1] = Num<T>::from_f32(v * c[k] + u * s[k]);
    }
    const int rest = rot - 2 * half;
    if (rest > 0 && q_out != q)
        for (int i = threadIdx.x; i < heads * rest; i += blockDim.x) {
            const int h = i / rest, k = 2 * half + i % rest;
            q_out[((size_t)t * heads + h) * qo_head_dim + qo_rot0 + k] = q[((size_t)t * heads + h) * q_head_dim + q_rot0 + k];
        }
}

OXR_API int oxr_latent_prep(void* pool, long long slot_stride, long long pool_slots, const void* down, int rank, int rot, const float* weight, float eps,
                            const void* q, int heads, int q_head_dim, int q_rot0, void* q_out, int qo_head_dim, int qo_rot0, const float* cos_t,
                            const float* sin_t, int half, const int* slots, int n_tokens, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rot < 0 || 2 * half > rot || q_rot0 + rot > q_head_dim || qo_rot0 + rot > qo_head_dim) return OXR_BAD_ARGUMENT;
    if (dtype == 0)
        latent_prep_kernel<float><<<n_tokens, 128, 0, stream>>>((float*)pool, slot_stride, pool_slots, (const float*)down, rank, rot, weight, eps, (const float*)q, heads,
                                                               q_head_dim, q_rot0, (float*)q_out, qo_head_dim, qo_rot0, cos_t, sin_t, half, slots, status);
    else
        latent_prep_kernel<__nv_bfloat16><<<n_tokens, 128, 0, stream>>>((__nv_bfloat16*)pool, slot_stride, pool_slots, (const __nv_bfloat16*)down, rank, rot, weight,
                                                                       eps, (const __nv_bfloat16*)q, heads, q_head_dim, q_rot0, (__nv_bfloat16*)q_out, qo_head_dim,
                                                                       qo_rot0, cos_t, sin_t, half, slots, status);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- per-head linear map
// out[t, h, out0 + o] = sum_i x[t, h, x0 + i] * w[h, i, o]   (w stored input-major per head: [heads, n_in, n_out]); fp32 sums in the
// order i = 0, 1, 2, ...; entries of out outside [out0, out0 + n_out) are left alone. grid (token tiles, heads).
template <typename T, int TM>
__global__ void __launch_bounds__(128) head_linear_kernel(T* __restrict__ out, int out_head_stride, int out0, const T* __restrict__ x, int x_head_stride,
                                                          int x0, const T* __restrict__ w, int n_in, int n_out, int heads, int n_tokens) {
    extern __shared__ float xs[];   // [TM, n_in]
    const int h = blockIdx.y, t0 = blockIdx.x * TM;
    for (int i = threadIdx.x; i < TM * n_in; i += blockDim.x) {
        const int m = i / n_in, k = i % n_in;
        xs[i] = (t0 + m < n_tokens) ? Num<T>::to_f32(x[((size_t)(t0 + m) * heads + h) * x_head_stride + x0 + k]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * n_in * n_out;
    for (int o = threadIdx.x; o < n_out; o += blockDim.x) {
        float acc[TM];
#pragma unroll
        for (int m = 0; m < TM; ++m) acc[m] = 0.f;
        for (int k = 0; k < n_in; ++k) {
            const float wv = Num<T>::to_f32(wh[(size_t)k * n_out + o]);
#pragma unroll
            for (int m = 0; m < TM; ++m) acc[m] = fmaf(xs[m * n_in + k], wv, acc[m]);
        }
#pragma unroll
        for (int m = 0; m < TM; ++m)
            if (t0 + m < n_tokens) out[((size_t)(t0 + m) * heads + h) * out_head_stride + out0 + o] = Num<T>::from_f32(acc[m]);
    }
}

// The same on the tensor cores (bf16, fp32 sums in k order per 16-wide step): a block takes 64 tokens of one head, a warp 16 of them;
// x rows and the head's matrix, 64 output columns at a time, stand in shared memory. n_in a multiple of 16, n_out of 16.
__device__ __forceinline__ void hl_ldsm_x4(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void hl_ldsm_x4_trans(uint32_t (&r)[4], const __nv_bfloat16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void hl_mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int HL_BM = 64, HL_BN = 64;

__global__ void __launch_bounds__(128) head_linear_mma_kernel(__nv_bfloat16* __restrict__ out, int out_head_stride, int out0,
                                                              const __nv_bfloat16* __restrict__ x, int x_head_stride, int x0,
                                                              const __nv_bfloat16* __restrict__ w, int n_in, int n_out, int heads, int n_tokens) {
    extern __shared__ __align__(16) unsigned char hl_smem[];
    const int lda = n_in + 8, ldb = HL_BN + 8;
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(hl_smem);   // [64][n_in + 8]
    __nv_bfloat16* Bs = As + HL_BM * lda;                            // [n_in][64 + 8]
    const int h = blockIdx.y, t0 = blockIdx.x * HL_BM, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < HL_BM * n_in; i += 128) {
        const int m = i / n_in, k = i % n_in;
        As[m * lda + k] = (t0 + m < n_tokens) ? x[((size_t)(t0 + m) * heads + h) * x_head_stride + x0 + k] : __float2bfloat16_rn(0.f);
    }
    const __nv_bfloat16* wh = w + (size_t)h * n_in * n_out;
    for (int c0 = 0; c0 < n_out; c0 += HL_BN) {
        const int cols = min(HL_BN, n_out - c0);
        __syncthreads();   // As is in; the previous chunk's Bs is no longer read
        for (int i = threadIdx.x; i < n_in * HL_BN; i += 128) {
            const int k = i / HL_BN, c = i % HL_BN;
            Bs[k * ldb + c] = c < cols ? wh[(size_t)k * n_out + c0 + c] : __float2bfloat16_rn(0.f);
        }
        __syncthreads();
        float acc[HL_BN / 8][4];
#pragma unroll
        for (int i = 0; i < HL_BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        for (int kk = 0; kk < n_in / 16; ++kk) {
            uint32_t a[4];
            hl_ldsm_x4(a, As + (warp * 16 + (lane & 15)) * lda + kk * 16 + 8 * (lane >> 4));
#pragma unroll
            for (int np = 0; np < HL_BN / 16; ++np) {
                uint32_t b[4];
                hl_ldsm_x4_trans(b, Bs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldb + np * 16 + 8 * (lane >> 4));
                hl_mma16816(acc[2 * np], a, b[0], b[1]);
                hl_mma16816(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int t = t0 + warp * 16 + (lane >> 2) + 8 * r;
            if (t >= n_tokens) continue;
            __nv_bfloat16* dst = out + ((size_t)t * heads + h) * out_head_stride + out0 + c0 + 2 * (lane & 3);
#pragma unroll
            for (int i = 0; i < HL_BN / 8; ++i)
                if (i * 8 + 2 * (lane & 3) < cols) {
                    dst[i * 8] = __float2bfloat16_rn(acc[i][2 * r]);
                    dst[i * 8 + 1] = __float2bfloat16_rn(acc[i][2 * r + 1]);
                }
        }
    }
}

OXR_API int oxr_head_linear(void* out, int out_head_stride, int out0, const void* x, int x_head_stride, int x0, const void* w, int n_in, int n_out,
                            int heads, int n_tokens, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_in <= 0 || n_out <= 0 || heads <= 0 || heads > 65535) return OXR_BAD_ARGUMENT;
    const size_t mma_smem = ((size_t)HL_BM * (n_in + 8) + (size_t)n_in * (HL_BN + 8)) * sizeof(__nv_bfloat16);
    if (dtype == 1 && n_tokens > 16 && n_in % 16 == 0 && n_out % 16 == 0 && mma_smem <= 200 * 1024) {
        static size_t configured = 0;
        if (mma_smem > 48 * 1024 && mma_smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(head_linear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem);
            if (e != cudaSuccess) return 1000 + (int)e;
            configured = mma_smem;
        }
        dim3 grid((n_tokens + HL_BM - 1) / HL_BM, heads);
        head_linear_mma_kernel<<<grid, 128, mma_smem, stream>>>((__nv_bfloat16*)out, out_head_stride, out0, (const __nv_bfloat16*)x, x_head_stride, x0,
                                                               (const __nv_bfloat16*)w, n_in, n_out, heads, n_tokens);
        return oxr_launch_status();
    }
    constexpr int TM = 8;
    const size_t smem = (size_t)TM * n_in * sizeof(float);
    if (smem > 48 * 1024) return OXR_BAD_ARGUMENT;
    dim3 grid((n_tokens + TM - 1) / TM, heads);
    if (dtype == 0)
        head_linear_kernel<float, TM><<<grid, 128, smem, stream>>>((float*)out, out_head_stride, out0, (const float*)x, x_head_stride, x0, (const float*)w, n_in,
                                                                  n_out, heads, n_tokens);
    else
        head_linear_kernel<__nv_bfloat16, TM><<<grid, 128, smem, stream>>>((__nv_bfloat16*)out, out_head_stride, out0, (const __nv_bfloat16*)x, x_head_stride, x0,
                                                                          (const __nv_bfloat16*)w, n_in, n_out, heads, n_tokens);
    return oxr_launch_status();
}
