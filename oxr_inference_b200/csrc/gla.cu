// Gated linear attention between its in- and out-projections: a recurrence whose state decays per key channel.
//
// Per request and head the state is a matrix S [DK, DV] (zero for a new request; one fp32 row per request holds S of every head). With
// a decay per key channel alpha_t = sigmoid(z_t)^(1 / tau), z_t = (the decay projection) + bias:
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          o_t = S_t^T q_t          q_t already scaled
//
// The decay (log-sigmoid, division by tau, exponential), S and every sum over it are fp32; T is the activation type of the q|k|v
// projections; z is fp32. The recurrence runs token by token in the order of the sequence whatever the cut, so a position's result does
// not depend on how a prompt was cut into steps. Columns of S (one value dimension each) are independent: a block takes 32 columns of one
// head of one request.
//
// grid (ceil(DV / 32), heads, requests); block = 32 * NW threads with NW = ceil(DK / KPT). Lane l owns the value column p = 32 blockIdx.x + l,
// warp w the key entries KPT w .. KPT w + KPT - 1: a thread keeps KPT = 32 or 16 entries of S in registers (16: twice the warps for the same
// state, which is what hides the loop's latencies when a step brings many tokens of a request; keys of up to 128). A tile of TT tokens goes through shared memory at
// a time (thread d brings entry d of k, q and the decay of each token; the next tile's loads are in flight while this one is computed); the
// warps' partial sums of S^T q meet in shared memory and are added in the order of the warps after the tile.
#include "common.cuh"

__device__ __forceinline__ float gla_log_sigmoid(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

template <typename T, int NW, int TT, int KPT>
__global__ void __launch_bounds__(32 * NW) gla_scan_kernel(
    float* __restrict__ y, const T* __restrict__ proj, int proj_stride, int q_col0, int k_col0, int v_col0, const float* __restrict__ z,
    const float* __restrict__ z_bias, float inv_tau, int heads, int DK, int DV, float q_scale, float* __restrict__ state, long long slot_stride,
    const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    constexpr int DKP = KPT * NW, NT = 32 * NW;      // NT >= DKP: thread d brings key entry d of every token
    __shared__ __align__(16) float ks[TT][DKP];
    __shared__ __align__(16) float qs[TT][DKP];
    __shared__ __align__(16) float as[TT][DKP];
    __shared__ float vs[TT][32], part[TT][NW][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n = threadIdx.x;
    const int p0 = blockIdx.x * 32, p = p0 + lane, h = blockIdx.y, r = blockIdx.z;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    float* S = state + (long long)state_slots[r] * slot_stride + (long long)h * DK * DV;
    const int n0 = KPT * warp;
    float s[KPT];
#pragma unroll
    for (int k = 0; k < KPT; ++k) s[k] = (n0 + k < DK && p < DV) ? S[(size_t)(n0 + k) * DV + p] : 0.f;
    const float zb = n < DK ? z_bias[h * DK + n] : 0.f;

    constexpr int VPT = (TT * 32 + NT - 1) / NT;      // v values per thread and tile
    T kreg[TT], qreg[TT], vreg[VPT];
    float zreg[TT];
    auto fetch = [&](int tile) {
        const int nt = min(TT, t1 - tile);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const bool ok = t < nt && n < DK;
            const size_t tok = (size_t)(tile + (t < nt ? t : 0));
            const T* row = proj + tok * proj_stride;
            kreg[t] = ok ? row[k_col0 + h * DK + n] : Num<T>::from_f32(0.f);
            qreg[t] = ok ? row[q_col0 + h * DK + n] : Num<T>::from_f32(0.f);
            zreg[t] = ok ? z[tok * heads * DK + h * DK + n] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = n + j * NT, t = i >> 5, c = i & 31;
            vreg[j] = (t < nt && p0 + c < DV) ? proj[(size_t)(tile + t) * proj_stride + v_col0 + h * DV + p0 + c] : Num<T>::from_f32(0.f);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (n < DKP) {
                ks[t][n] = Num<T>::to_f32(kreg[t]);
                qs[t][n] = Num<T>::to_f32(qreg[t]) * q_scale;
                as[t][n] = expf(gla_log_sigmoid(zreg[t] + zb) * inv_tau);
            }
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = n + j * NT;
            if (i < TT * 32) vs[i >> 5][i & 31] = Num<T>::to_f32(vreg[j]);
        }
    };
    fetch(t0);
    stash();
    __syncthreads();
    for (int tile = t0; tile < t1; tile += TT) {
        const int nt = min(TT, t1 - tile);
        const bool more = tile + TT < t1;
        if (more) fetch(tile + TT);
        for (int t = 0; t < nt; ++t) {
            const float tv = vs[t][lane];
            const float4* k4 = reinterpret_cast<const float4*>(&ks[t][n0]);
            const float4* q4 = reinterpret_cast<const float4*>(&qs[t][n0]);
            const float4* a4 = reinterpret_cast<const float4*>(&as[t][n0]);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};   // four chains, added in a fixed order
#pragma unroll
            for (int j = 0; j < KPT / 4; ++j) {
                const float4 kk = k4[j], qq = q4[j], aa = a4[j];
                s[4 * j] = fmaf(aa.x, s[4 * j], tv * kk.x);
                sum[0] = fmaf(s[4 * j], qq.x, sum[0]);
                s[4 * j + 1] = fmaf(aa.y, s[4 * j + 1], tv * kk.y);
                sum[1] = fmaf(s[4 * j + 1], qq.y, sum[1]);
                s[4 * j + 2] = fmaf(aa.z, s[4 * j + 2], tv * kk.z);
                sum[2] = fmaf(s[4 * j + 2], qq.z, sum[2]);
                s[4 * j + 3] = fmaf(aa.w, s[4 * j + 3], tv * kk.w);
                sum[3] = fmaf(s[4 * j + 3], qq.w, sum[3]);
            }
            part[t][warp][lane] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
        }
        __syncthreads();
        for (int i = n; i < nt * 32; i += NT) {
            const int t = i >> 5, c = i & 31;
            if (p0 + c < DV) {
                float num = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) num += part[t][w][c];
                y[(size_t)(tile + t) * heads * DV + h * DV + p0 + c] = num;
            }
        }
        if (more) {
            __syncthreads();   // the tile's sums have been read
            stash();
            __syncthreads();
        }
    }
#pragma unroll
    for (int k = 0; k < KPT; ++k)
        if (n0 + k < DK && p < DV) S[(size_t)(n0 + k) * DV + p] = s[k];
}

OXR_API int oxr_gla_scan(float* y, const void* proj, int n_requests, int proj_stride, int q_col0, int k_col0, int v_col0, const float* z,
                         const float* z_bias, float tau, int heads, int DK, int DV, float q_scale, float* state, long long slot_stride, const int* cu_q,
                         const int* state_slots, int dtype, int key_entries_per_thread, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || DK <= 0 || DK > 256 || DV <= 0 || heads > 65535 || n_requests > 65535 || !(tau > 0.f)) return OXR_BAD_ARGUMENT;
    dim3 grid((DV + 31) / 32, heads, n_requests);
    // 16 key entries a thread (twice the warps per head) where that still fits a block of 8 warps; key_entries_per_thread 16 or 32 forces one
    const bool narrow = key_entries_per_thread == 16 ? DK <= 128 : (key_entries_per_thread == 32 ? false : DK <= 128);
    const int nw = narrow ? (DK + 15) / 16 : (DK + 31) / 32;
#define OXR_GLA(T, NW) \
    do { \
        if (narrow) gla_scan_kernel<T, NW, 8, 16><<<grid, 32 * NW, 0, stream>>>(y, (const T*)proj, proj_stride, q_col0, k_col0, v_col0, z, z_bias, 1.f / tau, \
                                                                                heads, DK, DV, q_scale, state, slot_stride, cu_q, state_slots); \
        else gla_scan_kernel<T, NW, 8, 32><<<grid, 32 * NW, 0, stream>>>(y, (const T*)proj, proj_stride, q_col0, k_col0, v_col0, z, z_bias, 1.f / tau, heads, \
                                                                         DK, DV, q_scale, state, slot_stride, cu_q, state_slots); \
    } while (0)
#define OXR_GLA_T(T) \
    do { \
        if (nw <= 1) OXR_GLA(T, 1); \
        else if (nw <= 2) OXR_GLA(T, 2); \
        else if (nw <= 4) OXR_GLA(T, 4); \
        else OXR_GLA(T, 8); \
    } while (0)
    if (dtype == 0) OXR_GLA_T(float);
    else OXR_GLA_T(__nv_bfloat16);
#undef OXR_GLA_T
#undef OXR_GLA
    return oxr_launch_status();
}
