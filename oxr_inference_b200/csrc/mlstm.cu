// The matrix-memory recurrence of xLSTM (mLSTM) between its in- and out-projections, and the per-head norm with its gate.
//
// Per request and head the state is a matrix S [DK, DV], a vector n [DK] and a running maximum m (all zero for a new
// request; one fp32 row per request: S of every head, then n of every head, then m of every head). With the log input gate
// a_t = cap tanh(zi_t / cap) and the log forget gate b_t = logsigmoid(cap tanh(zf_t / cap)) (zi, zf: the gate projections
// plus their biases):
//
//   m_t = max(b_t + m_(t-1), a_t)
//   S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T          n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      q_t already scaled by DK^(-1/2)
//
// Two kernels: the tokens' gates (activations, the running maximum, the three exponentials each token needs), then the
// recurrence over the state. Gates, exponentials, S, n, m and every sum over them are fp32; T is the activation type of the
// q|k|v projections.
// The recurrence runs token by token in the order of the sequence whatever the cut, so a position's result does not
// depend on how a prompt was cut into steps. Columns of S (one value dimension each) are independent: a block takes 32
// columns of one head of one request; n and m are the same in all blocks of a head, and the first one writes them back.
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid_f32(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

// The gates of a step's tokens, before the recurrence: one warp per (head, request) works out, 32 tokens at a time, the two
// activations side by side, then the running maximum m_t one token after the other (the only part of the mixer that is serial in
// the tokens and not in the state: a few operations a token), then side by side again the three numbers the recurrence needs of
// each token: exp(b_t + m_(t-1) - m_t), exp(a_t - m_t) and exp(-m_t). The request's m is read from its state row and left there
// as it stands after the request's last token.
__global__ void __launch_bounds__(32) mlstm_gates_kernel(float* __restrict__ coef, const float* __restrict__ gates, const float* __restrict__ gate_bias,
                                                        int heads, int DK, int DV, float cap, float* __restrict__ state, long long slot_stride,
                                                        const int* __restrict__ cu_q, const int* __restrict__ state_slots) {
    const int lane = threadIdx.x, h = blockIdx.x, r = blockIdx.y;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    float* mptr = state + (long long)state_slots[r] * slot_stride + (long long)heads * DK * DV + (long long)heads * DK + h;
    const float bias_i = gate_bias[h], bias_f = gate_bias[heads + h];
    float m = *mptr;
    for (int base = t0; base < t1; base += 32) {
        const int t = base + lane, count = min(32, t1 - base);
        float a = 0.f, b = 0.f;
        if (t < t1) {
            const float* g = gates + (size_t)t * 2 * heads;
            a = cap * tanhf((g[h] + bias_i) / cap);
            b = log_sigmoid_f32(cap * tanhf((g[heads + h] + bias_f) / cap));
        }
        float before = 0.f, mine = 0.f;
        for (int j = 0; j < count; ++j) {
            const float aj = __shfl_sync(0xffffffffu, a, j), bj = __shfl_sync(0xffffffffu, b, j);
            const float m_new = fmaxf(bj + m, aj);
            if (lane == j) { before = m; mine = m_new; }
            m = m_new;
        }
        if (t < t1) {
            float* out = coef + ((size_t)t * heads + h) * 3;
            out[0] = expf(b + before - mine);
            out[1] = expf(a - mine);
            out[2] = expf(-mine);
        }
    }
    if (lane == 0) *mptr = m;
}

// grid (ceil(DV / 32), heads, requests); block = 32 * NW threads with NW = ceil(DK / 32). Lane l owns the value column
// p = 32 blockIdx.x + l, warp w the key entries 32 w .. 32 w + 31: a thread keeps 32 entries of S in registers, and thread d
// entry d of n. A tile of TT tokens goes through shared memory at a time: k, q, v and the tokens' three gate numbers are loaded
// once per tile (the next tile's while this one is computed), the loop over tokens is multiply-adds only, the warps' partial sums of S^T q and of n . q meet in shared memory
// and are added in the order of the warps after the tile.
template <typename T, int NW, int TT>
__global__ void __launch_bounds__(32 * NW) mlstm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ proj, int proj_stride, int q_col0, int k_col0, int v_col0, const float* __restrict__ coef,
    int heads, int DK, int DV, float q_scale, float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots) {
    constexpr int KPT = 32, DKP = KPT * NW, NT = 32 * NW;
    __shared__ __align__(16) float ks[TT][DKP];
    __shared__ __align__(16) float qs[TT][DKP];
    __shared__ float vs[TT][32], part[TT][NW][32], partn[TT][NW], gc[TT][3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n = threadIdx.x;
    const int p0 = blockIdx.x * 32, p = p0 + lane, h = blockIdx.y, r = blockIdx.z;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t1 <= t0) return;
    float* slot = state + (long long)state_slots[r] * slot_stride;
    float* S = slot + (long long)h * DK * DV;
    float* nvec = slot + (long long)heads * DK * DV + (long long)h * DK;
    const int n0 = KPT * warp;
    float s[KPT];
#pragma unroll
    for (int k = 0; k < KPT; ++k) s[k] = (n0 + k < DK && p < DV) ? S[(size_t)(n0 + k) * DV + p] : 0.f;
    float nn = n < DK ? nvec[n] : 0.f;       // thread d keeps n[d]

    // A tile's inputs are fetched into registers while the tile before it is computed (all loads of a tile are issued back to back:
    // one trip to memory per tile, hidden behind the sums), then written to shared memory between two barriers.
    constexpr int VPT = (TT * 32 + NT - 1) / NT;      // v values per thread and tile
    T kreg[TT], qreg[TT], vreg[VPT];
    float creg = 0.f;
    auto fetch = [&](int tile) {
        const int nt = min(TT, t1 - tile);
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const bool ok = t < nt && n < DK;
            const T* row = proj + (size_t)(tile + (t < nt ? t : 0)) * proj_stride;
            kreg[t] = ok ? row[k_col0 + h * DK + n] : Num<T>::from_f32(0.f);
            qreg[t] = ok ? row[q_col0 + h * DK + n] : Num<T>::from_f32(0.f);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = n + j * NT, t = i >> 5, c = i & 31;
            vreg[j] = (t < nt && p0 + c < DV) ? proj[(size_t)(tile + t) * proj_stride + v_col0 + h * DV + p0 + c] : Num<T>::from_f32(0.f);
        }
        if (n < nt * 3) creg = coef[((size_t)(tile + n / 3) * heads + h) * 3 + n % 3];
    };
    auto stash = [&]() {
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            ks[t][n] = Num<T>::to_f32(kreg[t]);
            qs[t][n] = Num<T>::to_f32(qreg[t]) * q_scale;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = n + j * NT;
            if (i < TT * 32) vs[i >> 5][i & 31] = Num<T>::to_f32(vreg[j]);
        }
        if (n < TT * 3) gc[n / 3][n % 3] = creg;
    };
    fetch(t0);
    stash();
    __syncthreads();
    for (int tile = t0; tile < t1; tile += TT) {
        const int nt = min(TT, t1 - tile);
        const bool more = tile + TT < t1;
        if (more) fetch(tile + TT);
        for (int t = 0; t < nt; ++t) {
            const float keep = gc[t][0], take = gc[t][1];
            nn = fmaf(keep, nn, take * ks[t][n]);
            const float nq = warp_sum(nn * qs[t][n]);
            const float tv = take * vs[t][lane];
            const float4* k4 = reinterpret_cast<const float4*>(&ks[t][n0]);
            const float4* q4 = reinterpret_cast<const float4*>(&qs[t][n0]);
            float sum[4] = {0.f, 0.f, 0.f, 0.f};   // four chains, added in a fixed order
#pragma unroll
            for (int j = 0; j < KPT / 4; ++j) {
                const float4 kk = k4[j], qq = q4[j];
                s[4 * j] = fmaf(keep, s[4 * j], tv * kk.x);
                sum[0] = fmaf(s[4 * j], qq.x, sum[0]);
                s[4 * j + 1] = fmaf(keep, s[4 * j + 1], tv * kk.y);
                sum[1] = fmaf(s[4 * j + 1], qq.y, sum[1]);
                s[4 * j + 2] = fmaf(keep, s[4 * j + 2], tv * kk.z);
                sum[2] = fmaf(s[4 * j + 2], qq.z, sum[2]);
                s[4 * j + 3] = fmaf(keep, s[4 * j + 3], tv * kk.w);
                sum[3] = fmaf(s[4 * j + 3], qq.w, sum[3]);
            }
            part[t][warp][lane] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            if (lane == 0) partn[t][warp] = nq;
        }
        __syncthreads();
        for (int i = n; i < nt * 32; i += NT) {
            const int t = i >> 5, c = i & 31;
            if (p0 + c < DV) {
                float num = 0.f, nq = 0.f;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    num += part[t][w][c];
                    nq += partn[t][w];
                }
                const float den = fmaxf(fabsf(nq), gc[t][2]) + 1e-6f;
                y[(size_t)(tile + t) * heads * DV + h * DV + p0 + c] = num / den;
            }
        }
        if (more) {
            __syncthreads();   // the tile's sums and gate numbers have been read
            stash();
            __syncthreads();
        }
    }
#pragma unroll
    for (int k = 0; k < KPT; ++k)
        if (n0 + k < DK && p < DV) S[(size_t)(n0 + k) * DV + p] = s[k];
    if (blockIdx.x == 0 && n < DK) nvec[n] = nn;
}

OXR_API int oxr_mlstm_scan(float* y, float* coef, const void* proj, int n_requests, int proj_stride, int q_col0, int k_col0, int v_col0,
                           const float* gates, const float* gate_bias, int heads, int DK, int DV, float cap, float q_scale, float* state,
                           long long slot_stride, const int* cu_q, const int* state_slots, int dtype, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || DK <= 0 || DK > 256 || DV <= 0 || heads > 65535 || n_requests > 65535 || !(cap > 0.f)) return OXR_BAD_ARGUMENT;
    mlstm_gates_kernel<<<dim3(heads, n_requests), 32, 0, stream>>>(coef, gates, gate_bias, heads, DK, DV, cap, state, slot_stride, cu_q, state_slots);
    dim3 grid((DV + 31) / 32, heads, n_requests);
    const int nw = (DK + 31) / 32;
#define OXR_MLSTM(T, NW) \
    mlstm_scan_kernel<T, NW, 8><<<grid, 32 * NW, 0, stream>>>(y, (const T*)proj, proj_stride, q_col0, k_col0, v_col0, coef, heads, DK, DV, q_scale, \
                                                             state, slot_stride, cu_q, state_slots)
#define OXR_MLSTM_T(T) \
    do { \
        if (nw <= 1) OXR_MLSTM(T, 1); \
        else if (nw <= 2) OXR_MLSTM(T, 2); \
        else if (nw <= 4) OXR_MLSTM(T, 4); \
        else OXR_MLSTM(T, 8); \
    } while (0)
    if (dtype == 0) OXR_MLSTM_T(float);
    else OXR_MLSTM_T(__nv_bfloat16);
#undef OXR_MLSTM_T
#undef OXR_MLSTM
    return oxr_launch_status();
}

// out[t, h, d] = y[t, h, d] / rms(y[t, h, :]) * weight[h, d] * act(gate[t, gate_col0 + h DV + d]) with act = sigmoid, or silu when `silu`;
// one warp per (token, head), everything in fp32, rounded once to T.
template <typename T>
__global__ void head_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, int gate_col0,
                                      const float* __restrict__ weight, int heads, int DV, float eps, int silu) {
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * warps + (threadIdx.x >> 5);
    if (h >= heads) return;
    const float* o = y + ((size_t)t * heads + h) * DV;
    float sq = 0.f;
    for (int d = lane; d < DV; d += 32) sq = fmaf(o[d], o[d], sq);
    const float inv = 1.f / sqrtf(warp_sum(sq) / (float)DV + eps);
    for (int d = lane; d < DV; d += 32) {
        const float g = Num<T>::to_f32(gate[(size_t)t * gate_stride + gate_col0 + h * DV + d]);
        out[((size_t)t * heads + h) * DV + d] = Num<T>::from_f32(o[d] * inv * weight[h * DV + d] * ((silu ? g : 1.f) / (1.f + expf(-g))));
    }
}

OXR_API int oxr_head_norm_gate(void* out, const float* y, const void* gate, int n_tokens, int gate_stride, int gate_col0, const float* weight,
                               int heads, int DV, float eps, int silu, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || DV <= 0) return OXR_BAD_ARGUMENT;
    const int warps = heads >= 4 ? 4 : heads;
    dim3 grid(n_tokens, (heads + warps - 1) / warps);
    if (grid.y > 65535) return OXR_BAD_ARGUMENT;
    if (dtype == 0) head_norm_gate_kernel<float><<<grid, 32 * warps, 0, stream>>>((float*)out, y, (const float*)gate, gate_stride, gate_col0, weight, heads, DV, eps, silu);
    else head_norm_gate_kernel<__nv_bfloat16><<<grid, 32 * warps, 0, stream>>>((__nv_bfloat16*)out, y, (const __nv_bfloat16*)gate, gate_stride, gate_col0, weight, heads, DV, eps, silu);
    return oxr_launch_status();
}
