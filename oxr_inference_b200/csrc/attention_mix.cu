// Paged attention whose heads talk to each other before the softmax, one block per query token, all arithmetic in fp32.
//
// For the query at position p of its request and every key j it sees (j <= p, within the last `window` keys when a window is given):
//
//   s_g(j)  = (q_g . k_kv(g)(j)) * scale                        for every query head g
//   s_g(j) <- cap * tanh(s_g(j) / cap)                          when cap > 0
//   s'_h(j) = sum_g mix[h, g] * s_g(j)                          when a mixing matrix [H, H] is given (else s' = s)
//   w_h(j)  = exp(s'_h(j)) / (sink + sum_j exp(s'_h(j)))         sink = 1 (a place with score 0 and no value) or 0
//   o_h     = sum_j w_h(j) * v_kv(h)(j)        then, with a gate, o_h <- o_h * sigmoid(gate_h)
//
// Because a head's weights depend on all heads' scores, a block computes all H heads of one token together: 32 keys at a time,
// the raw scores of all heads meet in shared memory, each warp mixes and normalises its heads (running maximum and sum), and
// every thread owns a few (head, value entry) sums. Keys are taken 32 at a time from the first visible one, so a row's result
// depends only on its position and the keys it sees, whatever the step holds. T is the type of q, of the cache and of the output.
//
// Also here: what stands between the q|k|v product and this kernel (biases, the rotation of entry pairs, the cache write).
#include "common.cuh"

template <typename T, int EPT>
__global__ void attn_mix_rows_kernel(
    T* __restrict__ out, const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, long long k_slot_stride, int k_head_stride,
    const T* __restrict__ v_pool, long long v_slot_stride, int v_head_stride, int DK, int DV, int H, int KVH, const int* __restrict__ positions,
    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_width, int page_size, int num_pages, float scale,
    float cap, const float* __restrict__ mix, int sink_one, int window, const T* __restrict__ gate, int gate_stride, int* status) {
    extern __shared__ __align__(16) unsigned char mix_smem[];
    long long* slots = reinterpret_cast<long long*>(mix_smem);   // [32]
    float* qs = reinterpret_cast<float*>(slots + 32);            // [H, DK]
    float* S = qs + (size_t)H * DK;                              // [H, 32] raw scores of the 32 keys at hand
    float* P = S + (size_t)H * 32;                               // [H, 32] their weights exp(s' - m)
    float* m_run = P + (size_t)H * 32;                           // [H] running maximum
    float* l_run = m_run + H;                                    // [H] running sum
    float* corr = l_run + H;                                     // [H] factor on what was summed before
    float* mx = corr + H;                                        // [H, H]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x, r = req_of_token[t], p = positions[t];
    const int per = H / KVH, total = H * DV;
    for (int i = threadIdx.x; i < H * DK; i += blockDim.x) qs[i] = Num<T>::to_f32(q[(size_t)t * q_stride + i]);
    if (mix != nullptr)
        for (int i = threadIdx.x; i < H * H; i += blockDim.x) mx[i] = mix[i];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        m_run[h] = sink_one ? 0.f : -INFINITY;   // the sink: a key with score 0
        l_run[h] = sink_one ? 1.f : 0.f;
    }
    float acc[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) acc[i] = 0.f;
    int lo = 0;
    if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
    const int* table = block_table + (size_t)r * table_width;
    __syncthreads();

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool seen = j <= p;
        if (warp == 0) {
            long long slot = -1;
            if (seen) {
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) oxr_report(status, OXR_BAD_PAGE, t);
                else slot = (long long)page * page_size + j % page_size;
            }
            slots[lane] = slot;
        }
        __syncthreads();
        const long long slot = slots[lane];
        for (int g = warp; g < H; g += warps) {
            float s = 0.f;
            if (slot >= 0) {
                const T* kr = k_pool + slot * k_slot_stride + (long long)(g / per) * k_head_stride;
                const float* qg = qs + (size_t)g * DK;
                float dot = 0.f;
                for (int d = 0; d < DK; ++d) dot = fmaf(qg[d], Num<T>::to_f32(kr[d]), dot);
                s = dot * scale;
                if (cap > 0.f) s = cap * tanhf(s / cap);
            }
            S[g * 32 + lane] = s;
        }
        __syncthreads();
        for (int h = warp; h < H; h += warps) {
            float s = -INFINITY;
            if (slot >= 0) {
                if (mix != nullptr) {
                    s = 0.f;
                    const float* row = mx + (size_t)h * H;
                    for (int g = 0; g < H; ++g) s = fmaf(row[g], S[g * 32 + lane], s);
                } else {
                    s = S[h * 32 + lane];
                }
            }
            const float m_old = m_run[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            float w = 0.f, c = 1.f;
            if (m_new != -INFINITY) {
                c = expf(m_old - m_new);             // m_old = -inf: 0
                w = slot >= 0 ? expf(s - m_new) : 0.f;
            }
            const float sum = warp_sum(w);
            P[h * 32 + lane] = w;
            __syncwarp();
            if (lane == 0) {
                corr[h] = c;
                m_run[h] = m_new;
                l_run[h] = l_run[h] * c + sum;
            }
        }
        __syncthreads();
        const int count = min(32, p - j0 + 1);
#pragma unroll
        for (int i = 0; i < EPT; ++i) {
            const int e = threadIdx.x + i * blockDim.x;
            if (e < total) {
                const int h = e / DV, d = e - h * DV;
                const float* ph = P + h * 32;
                float a = acc[i] * corr[h];
                const long long off = (long long)(h / per) * v_head_stride + d;
                for (int jj = 0; jj < count; ++jj) {
                    const long long sj = slots[jj];
                    if (sj >= 0) a = fmaf(ph[jj], Num<T>::to_f32(v_pool[sj * v_slot_stride + off]), a);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        if (e < total) {
            const int h = e / DV;
            const float l = l_run[h];
            float o = l > 0.f ? acc[i] / l : 0.f;
            if (gate != nullptr) o = o / (1.f + expf(-Num<T>::to_f32(gate[(size_t)t * gate_stride + e])));
            out[(size_t)t * total + e] = Num<T>::from_f32(o);
        }
    }
}

template <typename T, int EPT>
static int launch_mix_rows(void* out, const void* q, int q_stride, const void* k_pool, long long k_slot_stride, int k_head_stride, const void* v_pool,
                           long long v_slot_stride, int v_head_stride, int DK, int DV, int H, int KVH, int n_tokens, const int* positions,
                           const int* req_of_token, const int* block_table, int table_width, int page_size, int num_pages, float scale, float cap,
                           const float* mix, int sink_one, int window, const void* gate, int gate_stride, int* status, int threads, size_t smem,
                           cudaStream_t stream) {
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mix_rows_kernel<T, EPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = smem;
    }
    attn_mix_rows_kernel<T, EPT><<<n_tokens, threads, smem, stream>>>(
        (T*)out, (const T*)q, q_stride, (const T*)k_pool, k_slot_stride, k_head_stride, (const T*)v_pool, v_slot_stride, v_head_stride, DK, DV, H, KVH,
        positions, req_of_token, block_table, table_width, page_size, num_pages, scale, cap, mix, sink_one, window, (const T*)gate, gate_stride, status);
    return oxr_launch_status();
}

OXR_API int oxr_attention_mix_rows(void* out, const void* q, int q_stride, const void* k_pool, long long k_slot_stride, int k_head_stride,
                                   const void* v_pool, long long v_slot_stride, int v_head_stride, int DK, int DV, int H, int KVH, int n_tokens,
                                   const int* positions, const int* req_of_token, const int* block_table, int table_width, int page_size,
                                   int num_pages, float scale, float cap, const float* mix, int sink_one, int window, const void* gate,
                                   int gate_stride, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (DK <= 0 || DV <= 0 || H <= 0 || KVH <= 0 || H % KVH || page_size <= 0 || window < 0 || cap < 0.f) return OXR_BAD_ARGUMENT;
    const int total = H * DV;
    const int threads = total <= 512 ? 128 : 256;
    const int each = (total + threads - 1) / threads;
    const size_t smem = 32 * sizeof(long long) + ((size_t)H * DK + 2 * (size_t)H * 32 + 3 * (size_t)H + (size_t)H * H) * sizeof(float);
    if (smem > 200 * 1024 || each > 128) return OXR_BAD_ARGUMENT;
#define OXR_MIX(T, EPT) \
    return launch_mix_rows<T, EPT>(out, q, q_stride, k_pool, k_slot_stride, k_head_stride, v_pool, v_slot_stride, v_head_stride, DK, DV, H, KVH, n_tokens, \
                                   positions, req_of_token, block_table, table_width, page_size, num_pages, scale, cap, mix, sink_one, window, gate, \
                                   gate_stride, status, threads, smem, stream)
    if (dtype == 0) {
        if (each <= 4) OXR_MIX(float, 4);
        if (each <= 16) OXR_MIX(float, 16);
        if (each <= 48) OXR_MIX(float, 48);
        OXR_MIX(float, 128);
    }
    if (each <= 4) OXR_MIX(__nv_bfloat16, 4);
    if (each <= 16) OXR_MIX(__nv_bfloat16, 16);
    if (each <= 48) OXR_MIX(__nv_bfloat16, 48);
    OXR_MIX(__nv_bfloat16, 128);
#undef OXR_MIX
}

// ---------------------------------------------------------------------------------------------- between the product and attention
// One block per token. proj[t] = [q (cq) | k (ck) | v (cv) | ...] as the stacked product left it:
//   every entry gets its bias (fp32, optional);
//   the first `rot` entries of every q and k head turn pair by pair: (u, v) = entries (2i, 2i+1) become
//   (u cos a_i - v sin a_i, v cos a_i + u sin a_i) with the token's angle i (cos/sin [tokens, rot / 2]); the rest pass;
//   q goes back in place, k and v go to pool[slot] (slot -1: not stored).
// All arithmetic fp32, each value rounded once.
template <typename T>
__global__ void bias_rope_store_kernel(T* __restrict__ proj, int proj_stride, int cq, int ck, int cv, int DK, const float* __restrict__ bias,
                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, long long pool_slots, const int* __restrict__ slots, int* status) {
    const int t = blockIdx.x;
    T* row = proj + (size_t)t * proj_stride;
    int slot = slots[t];
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) oxr_report(status, OXR_BAD_SLOT, t);
        slot = -1;
    }
    const float* c = cos_t + (size_t)t * half;
    const float* s = sin_t + (size_t)t * half;
    // a head is `half` pairs followed by DK - 2 half single entries: one thread per pair or single entry
    const int units = DK - half, n_units = (cq + ck) / DK * units;
    for (int i = threadIdx.x; i < n_units; i += blockDim.x) {
        const int head = i / units, unit = i - head * units;
        const bool pair = unit < half;
        const int col = head * DK + (pair ? 2 * unit : unit + half);
        float u = Num<T>::to_f32(row[col]), v = pair ? Num<T>::to_f32(row[col + 1]) : 0.f;
        if (bias != nullptr) { u += bias[col]; if (pair) v += bias[col + 1]; }
        if (pair) {
            const float cc = c[unit], ss = s[unit];
            const float u2 = u * cc - v * ss, v2 = v * cc + u * ss;
            u = u2; v = v2;
        }
        T* dst = col < cq ? row + col : (slot >= 0 ? k_pool + (long long)slot * ck + (col - cq) : nullptr);
        if (dst != nullptr) {
            dst[0] = Num<T>::from_f32(u);
            if (pair) dst[1] = Num<T>::from_f32(v);
        }
    }
    if (slot >= 0)
        for (int i = threadIdx.x; i < cv; i += blockDim.x) {
            float v = Num<T>::to_f32(row[cq + ck + i]);
            if (bias != nullptr) v += bias[cq + ck + i];
            v_pool[(long long)slot * cv + i] = Num<T>::from_f32(v);
        }
}

OXR_API int oxr_bias_rope_store(void* proj, int proj_stride, int cq, int ck, int cv, int DK, const float* bias, const float* cos_t, const float* sin_t,
                                int half, void* k_pool, void* v_pool, long long pool_slots, const int* slots, int n_tokens, int dtype, int* status,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (DK <= 0 || cq % DK || ck % DK || 2 * half > DK || half < 0 || cq + ck + cv > proj_stride) return OXR_BAD_ARGUMENT;
    if (dtype == 0)
        bias_rope_store_kernel<float><<<n_tokens, 256, 0, stream>>>((float*)proj, proj_stride, cq, ck, cv, DK, bias, cos_t, sin_t, half, (float*)k_pool,
                                                                   (float*)v_pool, pool_slots, slots, status);
    else
        bias_rope_store_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>((__nv_bfloat16*)proj, proj_stride, cq, ck, cv, DK, bias, cos_t, sin_t, half,
                                                                           (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, pool_slots, slots, status);
    return oxr_launch_status();
}
