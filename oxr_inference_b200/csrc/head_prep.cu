// What stands between the projections of an attention mixer and its attention kernel, for mixers whose heads pass any of: a bias, a
// short causal filter over time, an RMS norm (with a weight or without), a rotation of entry pairs (i, i + half) by per-token angles.
// One warp per (token, head); a head is a query head, a key head or a value head. Everything is computed in fp32 from the projections
// and rounded once: queries to `q_out`, keys and values to their cache rows.
//
//   u      = proj + bias                                            (what the filter's tail keeps: the projected value)
//   y_t    = sum_j taps[c, j] * u_(t - n + 1 + j)                    (n taps, the last on the current token; zeros before the sequence)
//   value  = y of the key head, when the values are the filtered keys (else the value projection, copied)
//   norm   = y / sqrt(mean(y^2) + eps) [* weight]                   before or after the rotation
//   rotate : (a, b) = (y_i, y_(i + half)) -> (a cos - b sin, b cos + a sin) for i < half, angles per token; the rest passes
//
// Earlier tokens of the same request are read from the step's own rows, tokens before the step from the request's tail (fp32, the last
// n - 1 projected values of every filtered channel, the oldest first, each a row of all channels); a second kernel moves the tails on
// after the step.
// Also here: the sigmoid gate on an attention output (per channel or per head), in place.
#include "common.cuh"

struct PrepArgs {
    int stride;              // elements per row of proj
    int q_col0, k_col0, v_col0;
    int H, KV, DK, DV;
    int has_k;               // 0: the mixer reads another layer's keys and values (queries only)
    int v_mode;              // 0: no values here; 1: the value projection is copied; 2: values are the filtered keys (DV == DK)
    const float* bias;       // [H DK + KV DK] for q then k, or null
    const float* taps;       // [channels, n_taps] or null, channels = H DK + KV DK (H DK for a mixer without keys)
    const float* taps_t;     // the same transposed, [n_taps, channels] (what the 16-byte kernel reads), or null
    int n_taps;
    int channels;
    float* tails;            // [slots, (n_taps - 1) * channels]: entry (j, c) is channel c's projected value n_taps - 1 - j tokens back; row stride tail_stride
    long long tail_stride;
    int norm;                // 0 none, 1 with weight, 2 without
    int norm_after;          // the norm comes after the rotation
    const float* q_weight;   // [DK]
    const float* k_weight;
    float eps;
    const float* cos_t;      // [tokens, half] or null
    const float* sin_t;
    int half;
    const int* slots;        // [tokens] cache slot of each token, -1: not stored
    long long pool_slots;
    const int* req_of_token;
    const int* cu_q;
    const int* state_slots;
    int* status;
};

template <typename T>
__global__ void __launch_bounds__(128) head_prep_kernel(T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                                        const T* __restrict__ proj, const PrepArgs a) {
    extern __shared__ float prep_smem[];   // [warps, max(DK, DV)]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x, head = blockIdx.y * warps + warp;
    const int n_k = a.has_k ? a.KV : 0, n_v = a.v_mode == 1 ? a.KV : 0;
    if (head >= a.H + n_k + n_v) return;
    const int slot = a.slots[t];
    const T* row = proj + (size_t)t * a.stride;
    if (head >= a.H + n_k) {   // a value head: copied to its cache row
        const int h = head - a.H - n_k;
        if (slot < 0) return;
        if (slot >= a.pool_slots) { if (lane == 0) oxr_report(a.status, OXR_BAD_SLOT, t); return; }
        T* dst = v_pool + ((long long)slot * a.KV + h) * a.DV;
        for (int d = lane; d < a.DV; d += 32) dst[d] = row[a.v_col0 + h * a.DV + d];
        return;
    }
    const bool is_q = head < a.H;
    const int h = is_q ? head : head - a.H;
    if (!is_q && slot < 0) return;   // a key nobody stores
    if (!is_q && slot >= a.pool_slots) { if (lane == 0) oxr_report(a.status, OXR_BAD_SLOT, t); return; }
    const int col0 = (is_q ? a.q_col0 : a.k_col0) + h * a.DK;      // in proj
    const int ch0 = (is_q ? 0 : a.H * a.DK) + h * a.DK;            // among the biased / filtered channels
    float* y = prep_smem + warp * max(a.DK, a.DV);
    const int r = a.req_of_token[t], step0 = a.cu_q[r], s = t - step0;
    const float* tail = a.taps != nullptr && a.n_taps > 1 ? a.tails + (long long)a.state_slots[r] * a.tail_stride : nullptr;
    float sq = 0.f;
    for (int d = lane; d < a.DK; d += 32) {
        const int c = ch0 + d;
        const float b = a.bias != nullptr ? a.bias[c] : 0.f;
        float v;
        if (a.taps == nullptr) {
            v = Num<T>::to_f32(row[col0 + d]) + b;
        } else {
            const float* w = a.taps + (size_t)c * a.n_taps;
            v = 0.f;
            for (int back = a.n_taps - 1; back >= 0; --back) {       // oldest first: the order of the sum does not depend on the cut
                float u;
                if (back <= s) u = Num<T>::to_f32(proj[(size_t)(t - back) * a.stride + col0 + d]) + b;
                else u = tail[(size_t)((a.n_taps - 1) - (back - s)) * a.channels + c];
                v = fmaf(w[a.n_taps - 1 - back], u, v);
            }
        }
        y[d] = v;
        sq = fmaf(v, v, sq);
    }
    __syncwarp();
    if (!is_q && a.v_mode == 2) {   // the values are the keys as they leave the filter
        T* dst = v_pool + ((long long)slot * a.KV + h) * a.DV;
        for (int d = lane; d < a.DV; d += 32) dst[d] = Num<T>::from_f32(y[d]);
    }
    const float* weight = is_q ? a.q_weight : a.k_weight;
    if (a.norm != 0 && !a.norm_after) {
        const float inv = 1.f / sqrtf(warp_sum(sq) / (float)a.DK + a.eps);
        for (int d = lane; d < a.DK; d += 32) y[d] = y[d] * inv * (a.norm == 1 ? weight[d] : 1.f);
        __syncwarp();
    }
    if (a.cos_t != nullptr) {
        const float* c = a.cos_t + (size_t)t * a.half;
        const float* sn = a.sin_t + (size_t)t * a.half;
        for (int i = lane; i < a.half; i += 32) {
            const float u = y[i], v = y[i + a.half];
            y[i] = u * c[i] - v * sn[i];
            y[i + a.half] = v * c[i] + u * sn[i];
        }
        __syncwarp();
    }
    float inv = 1.f;
    if (a.norm != 0 && a.norm_after) {
        float s2 = 0.f;
        for (int d = lane; d < a.DK; d += 32) s2 = fmaf(y[d], y[d], s2);
        inv = 1.f / sqrtf(warp_sum(s2) / (float)a.DK + a.eps);
    }
    T* dst = is_q ? q_out + ((size_t)t * a.H + h) * a.DK : k_pool + ((long long)slot * a.KV + h) * a.DK;
    for (int d = lane; d < a.DK; d += 32) dst[d] = Num<T>::from_f32(y[d] * inv * ((a.norm == 1 && a.norm_after) ? weight[d] : 1.f));
}

// The same for bf16 heads whose entries are whole 16-byte words (DK, DV, every column offset and the row stride multiples of 8, half a
// multiple of 8): DK / 8 neighbouring lanes take one head, each with eight entries in registers from the first load to the last store, so
// that every row moves as 16-byte words and nothing goes through shared memory; a warp takes as many heads as fit its 32 lanes. The
// rotation's partner entries come from the lane half / 8 further on (or back) by shuffles; the sums of squares are added over the head's
// lanes in lane order.
__device__ __forceinline__ void prep_unpack(const uint4& v, float (&out)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 prep_pack(const float (&v)[8]) {
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return out;
}
__device__ __forceinline__ void prep_load8(const float* p, float (&out)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
// sum of v over the `lph` lanes of this lane's head (lanes g0 .. g0 + lph - 1), in a fixed order; every lane of the warp calls it
__device__ __forceinline__ float prep_head_sum(float v, int g0, int lph) {
    if ((lph & (lph - 1)) == 0) {      // a power of two: the head's lanes are an aligned group, a butterfly stays inside it
        for (int o = lph >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    }
    float total = 0.f;
    for (int j = 0; j < lph; ++j) total += __shfl_sync(0xffffffffu, v, (g0 + j) & 31);
    return total;
}

__global__ void __launch_bounds__(128) head_prep_bf16x8_kernel(__nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool,
                                                               __nv_bfloat16* __restrict__ v_pool, const __nv_bfloat16* __restrict__ proj,
                                                               const PrepArgs a, int lph, int hpw) {
    using bf16 = __nv_bfloat16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int sub = lane / lph, l = lane - sub * lph, g0 = sub * lph;        // which head of the warp, which word of the head
    const int head = (blockIdx.y * warps + warp) * hpw + sub;
    const int n_k = a.has_k ? a.KV : 0, n_v = a.v_mode == 1 ? a.KV : 0;
    const int slot = a.slots[t];
    const bf16* row = proj + (size_t)t * a.stride;
    bool live = sub < hpw && head < a.H + n_k + n_v;
    const bool is_v = live && head >= a.H + n_k;
    if (is_v) {   // a value head: copied to its cache row
        const int h = head - a.H - n_k;
        if (slot >= a.pool_slots) { if (l == 0) oxr_report(a.status, OXR_BAD_SLOT, t); }
        else if (slot >= 0 && 8 * l < a.DV)
            *reinterpret_cast<uint4*>(v_pool + ((long long)slot * a.KV + h) * a.DV + 8 * l) = *reinterpret_cast<const uint4*>(row + a.v_col0 + h * a.DV + 8 * l);
        live = false;
    }
    const bool is_q = head < a.H;
    const int h = is_q ? head : head - a.H;
    if (live && !is_q && slot >= a.pool_slots) { if (l == 0) oxr_report(a.status, OXR_BAD_SLOT, t); live = false; }
    if (live && !is_q && slot < 0) live = false;       // a key nobody stores
    // lanes that are not live walk along with zeros: the shuffles below are for the whole warp
    const int col0 = (is_q ? a.q_col0 : a.k_col0) + h * a.DK + 8 * l;
    const int c0 = (is_q ? 0 : a.H * a.DK) + h * a.DK + 8 * l;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = 0.f;
    if (live) {
        float b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = 0.f;
        if (a.bias != nullptr) prep_load8(a.bias + c0, b);
        if (a.taps == nullptr) {
            prep_unpack(*reinterpret_cast<const uint4*>(row + col0), y);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] += b[i];
        } else {
            const int r = a.req_of_token[t], s = t - a.cu_q[r], keep = a.n_taps - 1;
            const float* tail = keep > 0 ? a.tails + (long long)a.state_slots[r] * a.tail_stride + c0 : nullptr;
            const float* w = a.taps_t + c0;
            for (int back = keep; back >= 0; --back) {       // oldest first: the order of the sum does not depend on the cut
                float u[8];
                if (back <= s) {
                    prep_unpack(*reinterpret_cast<const uint4*>(proj + (size_t)(t - back) * a.stride + col0), u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) u[i] += b[i];
                } else {
                    prep_load8(tail + (size_t)(keep - (back - s)) * a.channels, u);
                }
                float wj[8];
                prep_load8(w + (size_t)(keep - back) * a.channels, wj);
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = fmaf(wj[i], u[i], y[i]);
            }
        }
        if (!is_q && a.v_mode == 2)    // the values are the keys as they leave the filter
            *reinterpret_cast<uint4*>(v_pool + ((long long)slot * a.KV + h) * a.DV + 8 * l) = prep_pack(y);
    }
    const float* weight = is_q ? a.q_weight : a.k_weight;
    float wn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) wn[i] = 1.f;
    if (live && a.norm == 1) prep_load8(weight + 8 * l, wn);
    if (a.norm != 0 && !a.norm_after) {
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sq = fmaf(y[i], y[i], sq);
        const float inv = 1.f / sqrtf(prep_head_sum(sq, g0, lph) / (float)a.DK + a.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = y[i] * inv * wn[i];
    }
    if (a.cos_t != nullptr) {
        const int shift = a.half / 8;                        // lanes between an entry and its partner
        const bool lower = 8 * l < a.half, upper = !lower && 8 * l < 2 * a.half;
        float c[8], sn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { c[i] = 1.f; sn[i] = 0.f; }
        if (live && (lower || upper)) {
            const int at = lower ? 8 * l : 8 * l - a.half;
            prep_load8(a.cos_t + (size_t)t * a.half + at, c);
            prep_load8(a.sin_t + (size_t)t * a.half + at, sn);
        }
        const int partner = lower ? lane + shift : (upper ? lane - shift : lane);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_sync(0xffffffffu, y[i], partner & 31);
            // the lower entry u and the upper entry v of a pair become u cos - v sin and v cos + u sin
            y[i] = lower ? y[i] * c[i] - other * sn[i] : (upper ? y[i] * c[i] + other * sn[i] : y[i]);
        }
    }
    if (a.norm != 0 && a.norm_after) {
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) sq = fmaf(y[i], y[i], sq);
        const float inv = 1.f / sqrtf(prep_head_sum(sq, g0, lph) / (float)a.DK + a.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = y[i] * inv * wn[i];
    }
    if (live) {
        bf16* dst = is_q ? q_out + ((size_t)t * a.H + h) * a.DK : k_pool + ((long long)slot * a.KV + h) * a.DK;
        *reinterpret_cast<uint4*>(dst + 8 * l) = prep_pack(y);
    }
}

// After the step: the tail of every request becomes the last n - 1 projected values (with bias) of each filtered channel. One thread per
// (request, channel); it reads the whole old tail before it writes.
template <typename T>
__global__ void prep_tail_kernel(const T* __restrict__ proj, const PrepArgs a, int channels, int n_requests) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_requests * channels) return;
    const int r = i / channels, c = i % channels;
    const int t0 = a.cu_q[r], n = a.cu_q[r + 1] - t0, keep = a.n_taps - 1;
    if (n <= 0) return;
    const int q_ch = a.H * a.DK;
    const int col = c < q_ch ? a.q_col0 + c : a.k_col0 + (c - q_ch);
    const float b = a.bias != nullptr ? a.bias[c] : 0.f;
    float* tail = a.tails + (long long)a.state_slots[r] * a.tail_stride + c;
    float old[16];
    for (int j = 0; j < keep; ++j) old[j] = tail[(size_t)j * channels];
    for (int j = 0; j < keep; ++j) {
        const int back = keep - j;                 // entry j holds the value `back` tokens before the next one
        tail[(size_t)j * channels] = back <= n ? Num<T>::to_f32(proj[(size_t)(t0 + n - back) * a.stride + col]) + b : old[j + n];
    }
}

OXR_API int oxr_head_prep(void* q_out, void* k_pool, void* v_pool, const void* proj, int n_tokens, int n_requests, int stride, int q_col0, int k_col0,
                          int v_col0, int H, int KV, int DK, int DV, int has_k, int v_mode, const float* bias, const float* taps, const float* taps_t, int n_taps, float* tails,
                          long long tail_stride, int norm, int norm_after, const float* q_weight, const float* k_weight, float eps, const float* cos_t,
                          const float* sin_t, int half, const int* slots, long long pool_slots, const int* req_of_token, const int* cu_q,
                          const int* state_slots, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || KV <= 0 || DK <= 0 || DV <= 0 || 2 * half > DK || (taps != nullptr && (n_taps < 1 || n_taps > 17)) || (v_mode == 2 && DV != DK) ||
        (taps != nullptr && n_taps > 1 && tails == nullptr) || (norm == 1 && (q_weight == nullptr || (has_k && k_weight == nullptr))))
        return OXR_BAD_ARGUMENT;
    PrepArgs a;
    a.stride = stride; a.q_col0 = q_col0; a.k_col0 = k_col0; a.v_col0 = v_col0; a.H = H; a.KV = KV; a.DK = DK; a.DV = DV; a.has_k = has_k;
    a.v_mode = has_k ? v_mode : 0; a.bias = bias; a.taps = taps; a.taps_t = taps_t; a.n_taps = taps != nullptr ? n_taps : 0; a.channels = H * DK + (has_k ? KV * DK : 0); a.tails = tails; a.tail_stride = tail_stride;
    a.norm = norm; a.norm_after = norm_after; a.q_weight = q_weight; a.k_weight = k_weight; a.eps = eps; a.cos_t = half > 0 ? cos_t : nullptr;
    a.sin_t = sin_t; a.half = half; a.slots = slots; a.pool_slots = pool_slots; a.req_of_token = req_of_token; a.cu_q = cu_q;
    a.state_slots = state_slots; a.status = status;
    const int heads = H + (has_k ? KV : 0) + (a.v_mode == 1 ? KV : 0);
    const int warps = heads >= 4 ? 4 : heads;
    dim3 grid(n_tokens, (heads + warps - 1) / warps);
    if (grid.y > 65535) return OXR_BAD_ARGUMENT;
    const size_t smem = (size_t)warps * (DK > DV ? DK : DV) * sizeof(float);
    if (smem > 48 * 1024) return OXR_BAD_ARGUMENT;
    const bool words = dtype == 1 && DK % 8 == 0 && DV % 8 == 0 && DK <= 256 && (v_mode != 1 || DV <= DK) && half % 8 == 0 && stride % 8 == 0 && q_col0 % 8 == 0 &&
                       k_col0 % 8 == 0 && v_col0 % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pool % 16 == 0 &&
                       (uintptr_t)v_pool % 16 == 0 && (uintptr_t)bias % 16 == 0 && (uintptr_t)q_weight % 16 == 0 && (uintptr_t)k_weight % 16 == 0 &&
                       (uintptr_t)cos_t % 16 == 0 && (uintptr_t)sin_t % 16 == 0 &&
                       (taps == nullptr || (taps_t != nullptr && (uintptr_t)taps_t % 16 == 0 && (n_taps < 2 || ((uintptr_t)tails % 16 == 0 && tail_stride % 4 == 0))));
    if (words) {
        const int lph = DK / 8, hpw = 32 / lph;
        const int per_block = 4 * hpw;
        dim3 vgrid(n_tokens, (heads + per_block - 1) / per_block);
        if (vgrid.y > 65535) return OXR_BAD_ARGUMENT;
        head_prep_bf16x8_kernel<<<vgrid, 128, 0, stream>>>((__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)proj, a, lph, hpw);
    } else if (dtype == 0) head_prep_kernel<float><<<grid, 32 * warps, smem, stream>>>((float*)q_out, (float*)k_pool, (float*)v_pool, (const float*)proj, a);
    else head_prep_kernel<__nv_bfloat16><<<grid, 32 * warps, smem, stream>>>((__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                                                                            (const __nv_bfloat16*)proj, a);
    if (a.taps != nullptr && a.n_taps > 1) {
        const int channels = a.channels;
        const int total = n_requests * channels;
        if (dtype == 0) prep_tail_kernel<float><<<(total + 127) / 128, 128, 0, stream>>>((const float*)proj, a, channels, n_requests);
        else prep_tail_kernel<__nv_bfloat16><<<(total + 127) / 128, 128, 0, stream>>>((const __nv_bfloat16*)proj, a, channels, n_requests);
    }
    return oxr_launch_status();
}

// o[t, h DV + d] *= sigmoid(g[t, g_col0 + (per_head ? h : h DV + d)]) in place; the sigmoid in fp32.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, const T* __restrict__ g, int g_stride, int g_col0, int inner, int DV, int per_head, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / inner;
    const int c = (int)(i - t * inner);
    const float z = Num<T>::to_f32(g[t * g_stride + g_col0 + (per_head ? c / DV : c)]);
    o[i] = Num<T>::from_f32(Num<T>::to_f32(o[i]) / (1.f + expf(-z)));
}

// The same for bf16 rows of whole 16-byte words: eight entries per thread (a head's entries share their gate when it is per head).
__global__ void sigmoid_gate_bf16x8_kernel(__nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ g, int g_stride, int g_col0, int inner, int DV,
                                           int per_head, size_t words) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    const int per_row = inner / 8;
    const size_t t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    float v[8], z[8];
    prep_unpack(*reinterpret_cast<const uint4*>(o + t * inner + c), v);
    if (per_head) {
        const float zz = __bfloat162float(g[t * g_stride + g_col0 + c / DV]);
#pragma unroll
        for (int k = 0; k < 8; ++k) z[k] = zz;
    } else {
        prep_unpack(*reinterpret_cast<const uint4*>(g + t * g_stride + g_col0 + c), z);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = v[k] / (1.f + expf(-z[k]));
    *reinterpret_cast<uint4*>(o + t * inner + c) = prep_pack(v);
}

OXR_API int oxr_sigmoid_gate(void* o, const void* g, int n_tokens, int g_stride, int g_col0, int inner, int DV, int per_head, int dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (inner <= 0 || DV <= 0 || inner % DV) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n_tokens * inner;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 1 && inner % 8 == 0 && DV % 8 == 0 && (per_head || (g_stride % 8 == 0 && g_col0 % 8 == 0 && (uintptr_t)g % 16 == 0)) && (uintptr_t)o % 16 == 0) {
        const size_t words = total / 8;
        sigmoid_gate_bf16x8_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)o, (const __nv_bfloat16*)g, g_stride, g_col0, inner, DV,
                                                                                        per_head, words);
        return oxr_launch_status();
    }
    if (dtype == 0) sigmoid_gate_kernel<float><<<blocks, 256, 0, stream>>>((float*)o, (const float*)g, g_stride, g_col0, inner, DV, per_head, total);
    else sigmoid_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)o, (const __nv_bfloat16*)g, g_stride, g_col0, inner, DV, per_head, total);
    return oxr_launch_status();
}
