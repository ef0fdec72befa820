// A feed-forward of routed experts: the router's choice per token, and the experts' activation with the choice applied.
//
// Router: scores s = sigmoid(z) of the fp32 router logits z [tokens, E]. The E experts form `groups` equal groups of
// neighbours; a group's score is the sum of its two largest s (of its only one, when groups hold one expert); only experts
// of the `keep` best groups can be chosen. The `top` allowed experts with the largest s are chosen (the lower index wins a
// tie); their weights are their s divided by the sum of the chosen s (+ 1e-20), times `scale`. All of it in fp32.
// Variants, each an argument: scores that are the softmax of z over all experts instead of sigmoids (score_kind 1); a group's
// score that is its largest s instead of the sum of its two largest (group_kind 1); weights that are the chosen s themselves,
// times `scale`, not divided by their sum (renorm 0).
//
// For steps of many tokens the experts run one after the other instead, each over the tokens that chose it (`expert_sort`, `gather_rows`,
// then per expert two products and the activation, then `combine_rows`): the work is then that of the chosen experts only.
//
// The choice leaves the kernel twice: as lists (expert ids and weights, [tokens, top]) and as a dense row per token
// (gate [tokens, E]: the weight of a chosen expert, 0 for the others). With the dense row the experts run as two
// products over ALL experts' stacked weights: u = h W_up^T [tokens, E ff], a = gate[expert of the column] act(u), and
// y = a W_down^T sums over experts inside the product's reduction; an expert that was not chosen adds exact zeros.
#include "common.cuh"

constexpr int ROUTE_MAX_TOP = 32;
constexpr int ROUTE_MAX_GROUPS = 64;

__global__ void route_kernel(float* __restrict__ gate, int* __restrict__ ids, float* __restrict__ wts, const float* __restrict__ z, int n_tokens,
                             int E, int top, int groups, int keep, float scale, int score_kind, int group_kind, int renorm) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens) return;
    float* row = gate + (size_t)t * E;          // scratch for the scores until the last pass
    const float* zr = z + (size_t)t * E;
    if (score_kind == 1) {
        float zmax = -INFINITY, den = 0.f;
        for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, zr[e]);
        for (int e = 0; e < E; ++e) { row[e] = expf(zr[e] - zmax); den += row[e]; }
        for (int e = 0; e < E; ++e) row[e] = row[e] / den;
    } else {
        for (int e = 0; e < E; ++e) row[e] = 1.f / (1.f + expf(-zr[e]));
    }
    unsigned long long allowed = ~0ull;        // one bit per group
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        float score[ROUTE_MAX_GROUPS];
        for (int g = 0; g < groups; ++g) {
            float a = -1.f, b = -1.f;           // the two largest of the group (scores are >= 0)
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = row[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            score[g] = group_kind == 1 ? a : a + (b >= 0.f ? b : 0.f);
        }
        allowed = 0ull;
        for (int i = 0; i < keep; ++i) {
            int best = -1;
            float best_v = -INFINITY;
            for (int g = 0; g < groups; ++g)
                if (!((allowed >> g) & 1ull) && score[g] > best_v) { best_v = score[g]; best = g; }
            if (best >= 0) allowed |= 1ull << best;
        }
    }
    int chosen[ROUTE_MAX_TOP];
    float chosen_s[ROUTE_MAX_TOP];
    float sum = 0.f;
    for (int i = 0; i < top; ++i) {
        int best = -1;
        float best_v = -INFINITY;
        for (int e = 0; e < E; ++e) {
            const float v = row[e];             // -1 once chosen
            if (v >= 0.f && ((allowed >> (e / per)) & 1ull) && v > best_v) { best_v = v; best = e; }
        }
        chosen[i] = best;
        chosen_s[i] = best >= 0 ? best_v : 0.f;
        if (best >= 0) { row[best] = -1.f; sum += best_v; }
    }
    const float norm = renorm ? scale / (sum + 1e-20f) : scale;
    for (int e = 0; e < E; ++e) row[e] = 0.f;
    for (int i = 0; i < top; ++i) {
        const float w = chosen_s[i] * norm;
        if (chosen[i] >= 0) row[chosen[i]] = w;
        ids[(size_t)t * top + i] = chosen[i];
        wts[(size_t)t * top + i] = w;
    }
}


// The same choice with one WARP per token (up to 256 experts and 32 groups): lane l scores the experts l, l + 32, ..., the scores
// meet in shared memory, lane g adds up group g's two largest, and every pick (of a group, then of an expert) is one warp-wide
// maximum in which the lower index wins a tie. A decode step's handful of tokens costs a few microseconds instead of a serial walk.
constexpr int ROUTE_WARP_MAX_E = 256;

__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

__global__ void __launch_bounds__(128) route_warp_kernel(float* __restrict__ gate, int* __restrict__ ids, float* __restrict__ wts, const float* __restrict__ z,
                                                        int n_tokens, int E, int top, int groups, int keep, float scale, int score_kind,
                                                        int group_kind, int renorm) {
    __shared__ float sc[4][ROUTE_WARP_MAX_E];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n_tokens) return;
    float* s = sc[warp];
    const int per = E / groups;
    if (score_kind == 1) {
        float zmax = -INFINITY, den = 0.f;
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[(size_t)t * E + e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) { s[e] = expf(z[(size_t)t * E + e] - zmax); den += s[e]; }
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) s[e] = s[e] / den;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-z[(size_t)t * E + e]));
    }
    __syncwarp();
    unsigned allowed = 0xffffffffu;            // one bit per group
    if (groups > 1 && keep < groups) {
        float score = -INFINITY;               // lane g: group g
        if (lane < groups) {
            float a = -1.f, b = -1.f;
            for (int e = lane * per; e < (lane + 1) * per; ++e) {
                const float v = s[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            score = group_kind == 1 ? a : a + (b >= 0.f ? b : 0.f);
        }
        allowed = 0u;
        for (int i = 0; i < keep; ++i) {
            float v = ((allowed >> lane) & 1u) ? -INFINITY : score;
            int idx = lane;
            warp_argmax(v, idx);
            allowed |= 1u << (idx & 31);
        }
    }
    float sum = 0.f, mine_s = 0.f;
    int mine = -1;                             // lane i keeps the i-th pick
    for (int i = 0; i < top; ++i) {
        float v = -INFINITY;
        int idx = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float x = s[e];              // -1 once chosen
            if (x >= 0.f && ((allowed >> (e / per)) & 1u) && x > v) { v = x; idx = e; }
        }
        warp_argmax(v, idx);
        if (idx >= E) { idx = -1; v = 0.f; }       // nothing left to pick (scores that are not numbers): no expert, no weight
        if (lane == i) { mine = idx; mine_s = v; }
        if (lane == 0 && idx >= 0) s[idx] = -1.f;
        sum += v;
        __syncwarp();
    }
    const float norm = renorm ? scale / (sum + 1e-20f) : scale;
    for (int e = lane; e < E; e += 32) gate[(size_t)t * E + e] = 0.f;
    __syncwarp();
    if (lane < top) {
        const float w = mine_s * norm;
        if (mine >= 0) gate[(size_t)t * E + mine] = w;
        ids[(size_t)t * top + lane] = mine;
        wts[(size_t)t * top + lane] = w;
    }
}

OXR_API int oxr_route(float* gate, int* ids, float* wts, const float* z, int n_tokens, int E, int top, int groups, int keep, float scale,
                      int score_kind, int group_kind, int renorm, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > ROUTE_MAX_TOP || groups <= 0 || groups > ROUTE_MAX_GROUPS || E % groups || keep <= 0 || keep > groups ||
        top > keep * (E / groups) || score_kind < 0 || score_kind > 1 || group_kind < 0 || group_kind > 1)
        return OXR_BAD_ARGUMENT;
    if (E <= ROUTE_WARP_MAX_E && groups <= 32)
        route_warp_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(gate, ids, wts, z, n_tokens, E, top, groups, keep, scale, score_kind, group_kind, renorm);
    else
        route_kernel<<<(n_tokens + 63) / 64, 64, 0, stream>>>(gate, ids, wts, z, n_tokens, E, top, groups, keep, scale, score_kind, group_kind, renorm);
    return oxr_launch_status();
}

// a[t, c] = gate[t, c / ff] * relu(u[t, c])^2 over the stacked columns of all experts; the product in fp32, rounded once.
template <typename T>
__global__ void gated_relu2_kernel(T* __restrict__ a, const T* __restrict__ u, const float* __restrict__ gate, size_t total, int cols, int ff, int E) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    const float g = gate != nullptr ? gate[t * E + c / ff] : 1.f;
    const float v = fmaxf(Num<T>::to_f32(u[i]), 0.f);
    a[i] = Num<T>::from_f32(g * (v * v));
}

// the same for bfloat16 with 16-byte accesses: 8 neighbouring columns of one expert (ff a multiple of 8)
__global__ void gated_relu2_bf16x8_kernel(__nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ u, const float* __restrict__ gate,
                                          size_t total8, int cols, int ff, int E) {
    const size_t i8 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i8 >= total8) return;
    const size_t i = i8 * 8, t = i / cols;
    const int c = (int)(i - t * cols);
    const float g = gate != nullptr ? gate[t * E + c / ff] : 1.f;
    uint4 raw = *reinterpret_cast<const uint4*>(u + i);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 f = __bfloat1622float2(p[k]);
        f.x = fmaxf(f.x, 0.f);
        f.y = fmaxf(f.y, 0.f);
        p[k] = __floats2bfloat162_rn(g * (f.x * f.x), g * (f.y * f.y));
    }
    *reinterpret_cast<uint4*>(a + i) = raw;
}

OXR_API int oxr_gated_relu2(void* a, const void* u, const float* gate, int n_tokens, int E, int ff, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || ff <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n_tokens * E * ff;
    if (dtype == 1 && ff % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)u % 16 == 0) {
        gated_relu2_bf16x8_kernel<<<(unsigned)((total / 8 + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)u, gate, total / 8,
                                                                                            E * ff, ff, E);
        return oxr_launch_status();
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) gated_relu2_kernel<float><<<blocks, 256, 0, stream>>>((float*)a, (const float*)u, gate, total, E * ff, ff, E);
    else gated_relu2_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)u, gate, total, E * ff, ff, E);
    return oxr_launch_status();
}

// The clamped gated unit over the stacked columns of all experts: gu[t] = E stretches [gate (ff) | up (ff)], one per expert;
// a[t, e ff + c] = gate_w[t, e] * g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate_w None: 1.
template <typename T>
__global__ void expert_clamped_glu_kernel(T* __restrict__ a, const T* __restrict__ gu, const float* __restrict__ gate_w, size_t total, int ff, int E,
                                          float alpha, float limit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cols = E * ff;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols), e = c / ff, k = c - e * ff;
    const float w = gate_w != nullptr ? gate_w[t * E + e] : 1.f;
    const T* src = gu + t * 2 * cols + (size_t)e * 2 * ff;
    const float g = fminf(Num<T>::to_f32(src[k]), limit);
    const float u = fminf(fmaxf(Num<T>::to_f32(src[ff + k]), -limit), limit);
    a[i] = Num<T>::from_f32(w * (g / (1.f + expf(-alpha * g)) * (u + 1.f)));
}

OXR_API int oxr_expert_clamped_glu(void* a, const void* gu, const float* gate_w, int n_tokens, int E, int ff, float alpha, float limit, int dtype,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || ff <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n_tokens * E * ff;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) expert_clamped_glu_kernel<float><<<blocks, 256, 0, stream>>>((float*)a, (const float*)gu, gate_w, total, ff, E, alpha, limit);
    else expert_clamped_glu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)gu, gate_w, total, ff, E, alpha, limit);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- tokens grouped by expert
// One block orders the (token, choice) pairs by expert: a histogram in shared memory, its running sum, then every pair takes the
// next free place of its expert (pairs of one expert end up in no particular order: each row's result does not depend on where
// in its expert's stretch it stands).
constexpr int SORT_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(1024) expert_sort_kernel(int* __restrict__ counts, int* __restrict__ order, int* __restrict__ place,
                                                          int* __restrict__ tile_group, const int* __restrict__ ids, int total, int E, int pad,
                                                          int capacity) {
    __shared__ int hist[SORT_MAX_EXPERTS], cursor[SORT_MAX_EXPERTS];
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    for (int i = threadIdx.x; i < capacity; i += blockDim.x) order[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = at;
            counts[e] = hist[e];
            const int end = at + (hist[e] + pad - 1) / pad * pad;      // every expert's stretch is padded to whole tiles of `pad` rows
            if (tile_group != nullptr)
                for (int tile = at / pad; tile < end / pad; ++tile) tile_group[tile] = e;
            at = end;
        }
        if (tile_group != nullptr)
            for (int tile = at / pad; tile < capacity / pad; ++tile) tile_group[tile] = -1;   // tiles nobody uses
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) {
            const int at = atomicAdd(&cursor[e], 1);
            order[at] = i;
            place[i] = at;
        } else {
            place[i] = -1;
        }
    }
}

// pad: every expert's stretch of the ordered list starts at a multiple of `pad` (places in between hold -1); capacity: length of `order`,
// at least total + E * (pad - 1) rounded up to a multiple of pad; tile_group (optional): which expert each tile of `pad` places belongs to.
OXR_API int oxr_expert_sort(int* counts, int* order, int* place, int* tile_group, const int* ids, int total, int E, int pad, int capacity,
                            cudaStream_t stream) {
    if (total <= 0) return 0;
    if (E <= 0 || E > SORT_MAX_EXPERTS || pad <= 0 || capacity % pad != 0 || capacity < total + (pad > 1 ? E * (pad - 1) : 0)) return OXR_BAD_ARGUMENT;
    expert_sort_kernel<<<1, 1024, 0, stream>>>(counts, order, place, tile_group, ids, total, E, pad, capacity);
    return oxr_launch_status();
}

// out[i] = x[order[i] / per_row] (zeros where order[i] is -1): 16-byte copies where the rows allow them
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ order, int width, int per_row) {
    const int from = order[blockIdx.x];          // -1: a padding place, filled with zeros
    const size_t dst = (size_t)blockIdx.x * width, src = (size_t)(from < 0 ? 0 : from / per_row) * width;
    if (from < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[dst + i] = Num<T>::from_f32(0.f);
        return;
    }
    const bool wide = (width * sizeof(T)) % 16 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)x & 15) == 0;
    if (wide) {
        const int4* s4 = reinterpret_cast<const int4*>(x + src);
        int4* d4 = reinterpret_cast<int4*>(out + dst);
        for (int i = threadIdx.x; i < (int)(width * sizeof(T) / 16); i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[dst + i] = x[src + i];
    }
}

OXR_API int oxr_gather_rows(void* out, const void* x, const int* order, int rows, int width, int per_row, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || per_row <= 0) return OXR_BAD_ARGUMENT;
    if (dtype == 0) gather_rows_kernel<float><<<rows, 128, 0, stream>>>((float*)out, (const float*)x, order, width, per_row);
    else gather_rows_kernel<__nv_bfloat16><<<rows, 128, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, order, width, per_row);
    return oxr_launch_status();
}

// out[t] = sum_j weights[t, j] * y[place[t top + j]], summed in fp32 in the order of j, rounded once
template <typename T>
__global__ void combine_rows_kernel(T* __restrict__ out, const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                    int top, int width) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int at = place[(size_t)t * top + j];
            if (at >= 0) acc = fmaf(weights[(size_t)t * top + j], Num<T>::to_f32(y[(size_t)at * width + c]), acc);
        }
        out[(size_t)t * width + c] = Num<T>::from_f32(acc);
    }
}

OXR_API int oxr_combine_rows(void* out, const void* y, const int* place, const float* weights, int n_tokens, int top, int width, int dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top <= 0 || width <= 0) return OXR_BAD_ARGUMENT;
    if (dtype == 0) combine_rows_kernel<float><<<n_tokens, 256, 0, stream>>>((float*)out, (const float*)y, place, weights, top, width);
    else combine_rows_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)y, place, weights, top, width);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- SiLU-gated experts
// The SiLU-gated unit over the stacked columns of all experts: gu[t] = E stretches [gate (ff) | up (ff)], one per expert. With the
// token's weight w = gate_w[t, e] for expert e (0: not chosen; gate_w None: 1):
//   on_input:  a[t, e ff + c] = silu(w g) * (w u)      the weight multiplies what the expert READS (W (w h) = w (W h))
//   else:      a[t, e ff + c] = w * silu(g) * u
template <typename T>
__global__ void expert_silu_glu_kernel(T* __restrict__ a, const T* __restrict__ gu, const float* __restrict__ gate_w, size_t total, int ff, int E,
                                       int on_input) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cols = E * ff;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols), e = c / ff, k = c - e * ff;
    const float w = gate_w != nullptr ? gate_w[t * E + e] : 1.f;
    const T* src = gu + t * 2 * cols + (size_t)e * 2 * ff;
    float g = Num<T>::to_f32(src[k]), u = Num<T>::to_f32(src[ff + k]), out;
    if (on_input) {
        g *= w;
        u *= w;
        out = g / (1.f + expf(-g)) * u;
    } else {
        out = w * (g / (1.f + expf(-g)) * u);
    }
    a[i] = Num<T>::from_f32(w == 0.f ? 0.f : out);
}

// The same for bf16 and expert widths that are whole 16-byte words: eight columns of one expert per thread.
__global__ void expert_silu_glu_bf16x8_kernel(__nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ gu, const float* __restrict__ gate_w,
                                              size_t words, int ff, int E, int on_input) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= words) return;
    const int cols = E * ff, per_row = cols / 8;
    const size_t t = i / per_row;
    const int c = (int)(i - t * per_row) * 8, e = c / ff, k = c - e * ff;
    const float w = gate_w != nullptr ? gate_w[t * E + e] : 1.f;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
        const __nv_bfloat16* src = gu + t * 2 * cols + (size_t)e * 2 * ff + k;
        const uint4 gw = *reinterpret_cast<const uint4*>(src), uw = *reinterpret_cast<const uint4*>(src + ff);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gw);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uw);
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
        const float wi = on_input ? w : 1.f, wo = on_input ? 1.f : w;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            const float gx = g.x * wi, gy = g.y * wi;
            o2[j] = __floats2bfloat162_rn(wo * (gx / (1.f + expf(-gx)) * (u.x * wi)), wo * (gy / (1.f + expf(-gy)) * (u.y * wi)));
        }
    }
    *reinterpret_cast<uint4*>(a + t * cols + c) = packed;
}

OXR_API int oxr_expert_silu_glu(void* a, const void* gu, const float* gate_w, int n_tokens, int E, int ff, int on_input, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || ff <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n_tokens * E * ff;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 1 && ff % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)gu % 16 == 0) {
        const size_t words = total / 8;
        expert_silu_glu_bf16x8_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)gu, gate_w, words, ff, E, on_input);
        return oxr_launch_status();
    }
    if (dtype == 0) expert_silu_glu_kernel<float><<<blocks, 256, 0, stream>>>((float*)a, (const float*)gu, gate_w, total, ff, E, on_input);
    else expert_silu_glu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)gu, gate_w, total, ff, E, on_input);
    return oxr_launch_status();
}

// x[place[p]] *= weights[p] for every (token, choice) pair p: rows gathered by expert, each scaled by its pair's weight (fp32 product,
// rounded once). One block per pair.
template <typename T>
__global__ void scale_placed_rows_kernel(T* __restrict__ x, const int* __restrict__ place, const float* __restrict__ weights, int hidden) {
    const int row = place[blockIdx.x];
    if (row < 0) return;
    const float w = weights[blockIdx.x];
    T* dst = x + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Num<T>::from_f32(Num<T>::to_f32(dst[i]) * w);
}

OXR_API int oxr_scale_placed_rows(void* x, const int* place, const float* weights, int pairs, int hidden, int dtype, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    if (dtype == 0) scale_placed_rows_kernel<float><<<pairs, 128, 0, stream>>>((float*)x, place, weights, hidden);
    else scale_placed_rows_kernel<__nv_bfloat16><<<pairs, 128, 0, stream>>>((__nv_bfloat16*)x, place, weights, hidden);
    return oxr_launch_status();
}

// y[t] += sigmoid(z[t]) * s[t]: a second feed-forward's result joins the first's, multiplied by one gate per token (z fp32 logits).
template <typename T>
__global__ void add_row_gated_kernel(T* __restrict__ y, const T* __restrict__ s, const float* __restrict__ z, int hidden, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float g = 1.f / (1.f + expf(-z[i / hidden]));
    y[i] = Num<T>::from_f32(Num<T>::to_f32(y[i]) + g * Num<T>::to_f32(s[i]));
}

OXR_API int oxr_add_row_gated(void* y, const void* s, const float* z, int n, int hidden, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n * hidden;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) add_row_gated_kernel<float><<<blocks, 256, 0, stream>>>((float*)y, (const float*)s, z, hidden, total);
    else add_row_gated_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)s, z, hidden, total);
    return oxr_launch_status();
}
