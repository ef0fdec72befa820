// Paged attention whose heads talk to each other before the softmax, bfloat16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
// The same function as attn_mix_rows_kernel (attention_mix.cu), for a tile of consecutive query tokens of one request:
//
//   s_g(i, j)  = cap * tanh((q_g(i) . k_kv(g)(j)) * scale / cap)        every query head g            (tensor cores, then fp32)
//   s'_h(i, j) = sum_g mix[h, g] * s_g(i, j)                            fp32 FMAs, through shared memory
//   o_h(i)     = sum_j softmax_j(s'_h(i, .))(j) * v_kv(h)(j)            weights fp32, rounded to bfloat16 for the product with V
//
// A head's weights need ALL heads' scores of the same (query, key), so one block owns every head of its queries. The rows of an
// MMA tile are (head of one key/value group, query) pairs: with `per` query heads per key/value head a 16-row tile holds
// R = 16 / per queries, row = head_in_group * R + query. Warp w = (key/value head c = w % KVH, query part w / KVH) owns one such
// tile: its keys and values are those of head c alone. Per block of 16 keys: every warp computes its tile's raw scores, caps them
// and writes them to shared memory; after a barrier every thread mixes, for the (row, column) places of its own accumulator
// fragment, the H heads' scores of that place; then the usual running maximum / sum and P V on its own fragment.
// K and V blocks of all key/value heads arrive by cp.async (zero-filled outside the visible range), K of the next block while
// this block is mixed and multiplied, V of this block while its scores are computed. Keys can be dealt to several blocks
// (split-KV); the pieces' (maximum, sum, unnormalised output) meet in attn_mix_combine_kernel. The unit sink (a key with score
// 0 and no value) and the sigmoid gate join where a row is normalised.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BN = 16;        // keys per block
constexpr int PADE = 8;       // 16 bytes of padding per shared-memory row: ldmatrix rows fall on different banks
constexpr int MAX_WARPS = 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled and gmem is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// a 16-byte word from shared memory by its 32-bit address: no generic-pointer arithmetic in the mixing loop
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
constexpr float LOG2E = 1.4426950408889634f;
// cap * tanh(x / cap) = cap - 2 cap / (exp(2 x / cap) + 1), with x = raw * scale and k2 = 2 * scale / cap * log2(e): absolute error of
// a few 1e-7 of cap everywhere, exact limits at both ends (exp = inf: cap; exp = 0: -cap)
__device__ __forceinline__ float capped(float raw, float k2, float cap) { return fmaf(-2.f * cap, rcp_fast(ex2_fast(raw * k2) + 1.f), cap); }

struct MixArgs {
    bf16* out;
    const bf16* q;
    int q_stride;
    const bf16* k_pool;
    const bf16* v_pool;
    int H, KVH, HP, QT, SQ;   // SQ: query rows per head in the score exchange (QT * R, or 1 when every tile is one token)
    const int* tile_req;
    const int* tile_tok0;
    const int* cu_q;
    const int* positions;
    const int* block_table;
    int table_width, page_size, num_pages;
    float scale, cap;
    const float* mix;
    int sink_one, window;
    const bf16* gate;
    int gate_stride;
    int splits;
    float* part_o;    // [tokens, splits, H * DV]
    float* part_ml;   // [tokens, splits, H, 2]
    int* status;
};

__host__ __device__ inline size_t mix_smem_bytes(int DK, int DV, int H, int KVH, int HP, int QT, int SQ) {
    const int BM = SQ, warps = KVH * QT;
    return (size_t)warps * 16 * (DK + PADE) * 2 + (size_t)KVH * BN * (DK + PADE) * 2 + (size_t)KVH * BN * (DV + PADE) * 2 +
           (size_t)HP * BM * BN * 4 + (size_t)H * HP * 4 + 2 * BN * sizeof(long long);
}

template <int DK, int DV>
__global__ void __launch_bounds__(MAX_WARPS * 32, 1) attn_mix_mma_kernel(const MixArgs p) {
    extern __shared__ __align__(16) unsigned char mix_mma_smem[];
    constexpr int LQ = DK + PADE, LV = DV + PADE;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int H = p.H, KVH = p.KVH, per = H / KVH, R = 16 / per, QT = p.QT, BM = QT * R, HP = p.HP, SQ = p.SQ;
    const int n_warps = KVH * QT;
    bf16* Qs = reinterpret_cast<bf16*>(mix_mma_smem);              // [warps][16][LQ]
    bf16* Ks = Qs + (size_t)n_warps * 16 * LQ;                     // [KVH][BN][LQ]
    bf16* Vs = Ks + (size_t)KVH * BN * LQ;                         // [KVH][BN][LV]
    float* Ss = reinterpret_cast<float*>(Vs + (size_t)KVH * BN * LV);   // [HP][SQ][BN], a thread's columns side by side
    float* Tm = Ss + (size_t)HP * SQ * BN;                         // [H][HP]: mix[h][g], zeros beyond g = H
    long long* slot_s = reinterpret_cast<long long*>(Tm + (size_t)H * HP);   // [2][BN]
    const bool has_mix = p.mix != nullptr;

    const int tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.y;   // a prompt's last tiles see the most keys: they start first
    const int req = p.tile_req[tile];
    const int t0 = p.cu_q[req] + p.tile_tok0[tile];
    const int nq = min(BM, p.cu_q[req + 1] - t0);
    const int pos0 = p.positions[t0];
    const int hi = pos0 + nq - 1;                                  // the last key any query of the tile sees
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;   // the first
    const int b_first = lo / BN, nb = hi / BN - b_first + 1;
    const int b_begin = b_first + (int)((long long)split * nb / p.splits);
    const int b_end = b_first + (int)((long long)(split + 1) * nb / p.splits);
    const int* table = p.block_table + (size_t)req * p.table_width;

    // this thread's two rows of its warp's tile, and what they stand for
    const int c = warp % KVH, qt = warp / KVH, quad = lane & 3;
    const int r_a = lane >> 2, r_b = r_a + 8;
    const int h_a = c * per + r_a / R, h_b = c * per + r_b / R;
    const int qq_a = qt * R + r_a % R, qq_b = qt * R + r_b % R;
    const bool valid_a = qq_a < nq, valid_b = qq_b < nq;
    const int pos_a = pos0 + qq_a, pos_b = pos0 + qq_b;
    const int lo_a = p.window > 0 ? pos_a - p.window + 1 : 0, lo_b = p.window > 0 ? pos_b - p.window + 1 : 0;
    const bool warp_active = qt * R < nq;

    auto slot_of = [&](int j) -> long long {
        if (j < lo || j > hi) return -1;
        const int idx = j / p.page_size;
        const int page = idx < p.table_width ? table[idx] : -1;
        if (page < 0 || page >= p.num_pages) {
            oxr_report(p.status, OXR_BAD_PAGE, t0);
            return -1;
        }
        return (long long)page * p.page_size + j % p.page_size;
    };
    // rows of all key/value heads for the BN keys whose slots are given: dst [KVH][BN][ld]. A warp takes a key: its row of KVH * width
    // entries is one run of memory.
    auto issue_rows = [&](bf16* dst, int ld, const bf16* pool, int width, const long long* slots) {
        const int shift = width == 128 ? 4 : 3, row_chunks = KVH << shift;   // 16-byte pieces per head row: 16 or 8
        for (int key = warp; key < BN; key += n_warps) {
            const long long s = slots[key];
            const bf16* src = pool + (s < 0 ? 0 : s) * (long long)(KVH * width);
            for (int j = lane; j < row_chunks; j += 32) {
                const int kc = j >> shift, ch = j & ((1 << shift) - 1);
                cp_async_16(dst + ((size_t)kc * BN + key) * ld + ch * 8, src + j * 8, s >= 0);
            }
        }
    };

    // ---- prologue: queries, the mixing matrix, the first block's slots and keys
    {
        const int cpr = DK / 8, total = n_warps * 16 * cpr;
        for (int i = tid; i < total; i += nthreads) {
            const int w = i / (16 * cpr), rem = i - w * 16 * cpr, r = rem / cpr, ch = rem - r * cpr;
            const int qq = (w / KVH) * R + r % R, h = (w % KVH) * per + r / R;
            const bool ok = qq < nq;
            cp_async_16(Qs + ((size_t)w * 16 + r) * LQ + ch * 8, p.q + (size_t)(t0 + (ok ? qq : 0)) * p.q_stride + h * DK + ch * 8, ok);
        }
        cp_async_commit();
        if (has_mix) {
            for (int i = tid; i < H * HP; i += nthreads) {
                const int h = i / HP, g = i - h * HP;
                Tm[i] = g < H ? p.mix[h * H + g] : 0.f;
            }
            for (int i = tid; i < (HP - H) * SQ * BN; i += nthreads) Ss[(size_t)H * SQ * BN + i] = 0.f;
        }
        if (tid < BN) slot_s[tid] = b_begin < b_end ? slot_of(b_begin * BN + tid) : -1;
        // A piece of the keys (few tiles, the GPU is not full: every wait for memory shows): ask for all of the piece's K and V rows
        // at once, so that the block-by-block copies find them in L2.
        if (p.splits > 1 && b_end - b_begin <= 32) {
            const int k_lines = KVH * DK * 2 / 128, v_lines = KVH * DV * 2 / 128, lines = k_lines + v_lines;
            for (int i = tid; i < (b_end - b_begin) * BN * lines; i += nthreads) {
                const int key = i / lines, line = i - key * lines;
                const long long sl = slot_of(b_begin * BN + key);
                if (sl < 0) continue;
                const bf16* at = line < k_lines ? p.k_pool + sl * (long long)(KVH * DK) + line * 64 : p.v_pool + sl * (long long)(KVH * DV) + (line - k_lines) * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(at));
            }
        }
    }
    __syncthreads();
    if (b_begin < b_end) issue_rows(Ks, LQ, p.k_pool, DK, slot_s);
    cp_async_commit();

    float o_acc[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const float k2 = p.cap > 0.f ? 2.f * p.scale / p.cap * LOG2E : 0.f;
    const int pos_min = pos0 + qt * R;   // the earliest position among this warp's queries

    for (int b = b_begin, it = 0; b < b_end; ++b, ++it) {
        const long long* cur = slot_s + (it & 1) * BN;
        long long* nxt = slot_s + ((it + 1) & 1) * BN;
        cp_async_wait<0>();
        __syncthreads();   // K of this block (and the queries) are here; every warp is past the last block's P V
        issue_rows(Vs, LV, p.v_pool, DV, cur);
        cp_async_commit();
        if (tid < BN) nxt[tid] = b + 1 < b_end ? slot_of((b + 1) * BN + tid) : -1;

        // ---- raw scores of this warp's tile: [16 rows] x [BN keys]
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        if (warp_active) {
            const bf16* q_at = Qs + ((size_t)warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LQ + 8 * (lane >> 4);
            const bf16* k_at = Ks + ((size_t)c * BN + (lane & 7) + 8 * (lane >> 4)) * LQ + 8 * ((lane >> 3) & 1);
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                uint32_t qa[4], kr[4];
                ldsm_x4(qa, q_at + ks * 16);
                ldsm_x4(kr, k_at + ks * 16);
                mma16816(s[0], qa, kr[0], kr[1]);
                mma16816(s[1], qa, kr[2], kr[3]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[i][e] = p.cap > 0.f ? capped(s[i][e], k2, p.cap) : s[i][e] * p.scale;
                }
            if (has_mix) {
                // place (quad, n-tile, e) of a row <-> key column n-tile * 8 + 2 * quad + e
                if (valid_a) *reinterpret_cast<float4*>(Ss + ((size_t)h_a * SQ + qq_a) * BN + quad * 4) = make_float4(s[0][0], s[0][1], s[1][0], s[1][1]);
                if (valid_b) *reinterpret_cast<float4*>(Ss + ((size_t)h_b * SQ + qq_b) * BN + quad * 4) = make_float4(s[0][2], s[0][3], s[1][2], s[1][3]);
            }
        }
        __syncthreads();   // every head's scores are in shared memory; nobody reads this block's K any more
        if (b + 1 < b_end) issue_rows(Ks, LQ, p.k_pool, DK, nxt);
        cp_async_commit();

        // sp[row a / b][n-tile * 2 + e]
        float sp[2][4];
        uint32_t pa[4] = {0u, 0u, 0u, 0u};
        if (warp_active) {
            if (has_mix) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sp[0][e] = sp[1][e] = 0.f;
                // rows of queries that the tile does not have are not exchanged: such a thread reads row 0 and its result is masked
                uint32_t ta = smem_u32(Tm + (size_t)h_a * HP), tb = smem_u32(Tm + (size_t)h_b * HP);
                uint32_t sa = smem_u32(Ss + (size_t)(valid_a ? qq_a : 0) * BN + quad * 4), sb = smem_u32(Ss + (size_t)(valid_b ? qq_b : 0) * BN + quad * 4);
                const bool same_q = qq_a == qq_b;   // the same for the whole warp (R <= 8)
                const uint32_t per_head = (uint32_t)(SQ * BN * sizeof(float));
                if (same_q) {   // both rows are the same query's: one word of scores serves both
                    for (int g0 = 0; g0 < HP; g0 += 4, ta += 16, tb += 16) {
                        const float4 ta4 = lds128(ta), tb4 = lds128(tb);
                        const float tav[4] = {ta4.x, ta4.y, ta4.z, ta4.w}, tbv[4] = {tb4.x, tb4.y, tb4.z, tb4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e, sa += per_head) {
                            const float4 sv = lds128(sa);
                            sp[0][0] = fmaf(tav[e], sv.x, sp[0][0]); sp[0][1] = fmaf(tav[e], sv.y, sp[0][1]);
                            sp[0][2] = fmaf(tav[e], sv.z, sp[0][2]); sp[0][3] = fmaf(tav[e], sv.w, sp[0][3]);
                            sp[1][0] = fmaf(tbv[e], sv.x, sp[1][0]); sp[1][1] = fmaf(tbv[e], sv.y, sp[1][1]);
                            sp[1][2] = fmaf(tbv[e], sv.z, sp[1][2]); sp[1][3] = fmaf(tbv[e], sv.w, sp[1][3]);
                        }
                    }
                } else {
                    for (int g0 = 0; g0 < HP; g0 += 4, ta += 16, tb += 16) {
                        const float4 ta4 = lds128(ta), tb4 = lds128(tb);
                        const float tav[4] = {ta4.x, ta4.y, ta4.z, ta4.w}, tbv[4] = {tb4.x, tb4.y, tb4.z, tb4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e, sa += per_head, sb += per_head) {
                            const float4 sav = lds128(sa), sbv = lds128(sb);
                            sp[0][0] = fmaf(tav[e], sav.x, sp[0][0]); sp[0][1] = fmaf(tav[e], sav.y, sp[0][1]);
                            sp[0][2] = fmaf(tav[e], sav.z, sp[0][2]); sp[0][3] = fmaf(tav[e], sav.w, sp[0][3]);
                            sp[1][0] = fmaf(tbv[e], sbv.x, sp[1][0]); sp[1][1] = fmaf(tbv[e], sbv.y, sp[1][1]);
                            sp[1][2] = fmaf(tbv[e], sbv.z, sp[1][2]); sp[1][3] = fmaf(tbv[e], sbv.w, sp[1][3]);
                        }
                    }
                }
            } else {
                sp[0][0] = s[0][0]; sp[0][1] = s[0][1]; sp[0][2] = s[1][0]; sp[0][3] = s[1][1];
                sp[1][0] = s[0][2]; sp[1][1] = s[0][3]; sp[1][2] = s[1][2]; sp[1][3] = s[1][3];
            }
            // ---- mask, running maximum and sum. A block that every row of the warp sees whole needs no mask (all but a tile's last
            // block or two, and a window's first).
            const bool whole = (qt + 1) * R <= nq && b * BN + BN - 1 <= pos_min && (p.window == 0 || b * BN > pos_min + R - 1 - p.window);
            bool see_a[4], see_b[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) see_a[e] = see_b[e] = true;
            if (!whole) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = b * BN + (e >> 1) * 8 + 2 * quad + (e & 1);
                    see_a[e] = valid_a && j <= pos_a && j >= lo_a;
                    see_b[e] = valid_b && j <= pos_b && j >= lo_b;
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (see_a[e]) mx_a = fmaxf(mx_a, sp[0][e]);
                if (see_b[e]) mx_b = fmaxf(mx_b, sp[1][e]);
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const bool moved = mn_a != m_a || mn_b != m_b;
            const float corr_a = mn_a == -INFINITY ? 1.f : ex2_fast((m_a - mn_a) * LOG2E), corr_b = mn_b == -INFINITY ? 1.f : ex2_fast((m_b - mn_b) * LOG2E);
            const float off_a = mn_a == -INFINITY ? 0.f : mn_a * LOG2E, off_b = mn_b == -INFINITY ? 0.f : mn_b * LOG2E;
            float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                sp[0][e] = see_a[e] ? ex2_fast(fmaf(sp[0][e], LOG2E, -off_a)) : 0.f;
                sp[1][e] = see_b[e] ? ex2_fast(fmaf(sp[1][e], LOG2E, -off_b)) : 0.f;
                sum_a += sp[0][e];
                sum_b += sp[1][e];
            }
            m_a = mn_a; m_b = mn_b;
            l_a = l_a * corr_a + sum_a;   // this thread's share of the row's sum; the quad's shares meet at the end
            l_b = l_b * corr_b + sum_b;
            if (__any_sync(0xffffffffu, moved)) {   // once the maxima have settled there is nothing to rescale
#pragma unroll
                for (int i = 0; i < DV / 8; ++i) {
                    o_acc[i][0] *= corr_a; o_acc[i][1] *= corr_a;
                    o_acc[i][2] *= corr_b; o_acc[i][3] *= corr_b;
                }
            }
            pa[0] = pack_bf16(sp[0][0], sp[0][1]); pa[1] = pack_bf16(sp[1][0], sp[1][1]);
            pa[2] = pack_bf16(sp[0][2], sp[0][3]); pa[3] = pack_bf16(sp[1][2], sp[1][3]);
        }
        cp_async_wait<1>();
        __syncthreads();   // V of this block is here; nobody reads this block's scores any more
        if (warp_active) {
            const bf16* v_at = Vs + ((size_t)c * BN + (lane & 7) + 8 * ((lane >> 3) & 1)) * LV + 8 * (lane >> 4);
#pragma unroll
            for (int n2 = 0; n2 < DV / 16; ++n2) {
                uint32_t vr[4];
                ldsm_x4_trans(vr, v_at + n2 * 16);
                mma16816(o_acc[2 * n2], pa, vr[0], vr[1]);
                mma16816(o_acc[2 * n2 + 1], pa, vr[2], vr[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (!warp_active) return;

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const int total = H * DV;
    if (p.splits == 1) {
        // normalise here: the sink joins the denominator as exp(0 - maximum), the gate multiplies the row
        float f_a = 0.f, f_b = 0.f;
        if (p.sink_one) {
            const float ma = fmaxf(m_a, 0.f), mb = fmaxf(m_b, 0.f);
            const float ca = m_a == -INFINITY ? 0.f : __expf(m_a - ma), cb = m_b == -INFINITY ? 0.f : __expf(m_b - mb);
            f_a = ca / (l_a * ca + __expf(-ma));
            f_b = cb / (l_b * cb + __expf(-mb));
        } else {
            f_a = l_a > 0.f ? 1.f / l_a : 0.f;
            f_b = l_b > 0.f ? 1.f / l_b : 0.f;
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            const int d = i * 8 + 2 * quad;
            if (valid_a) {
                float x = o_acc[i][0] * f_a, y = o_acc[i][1] * f_a;
                if (p.gate != nullptr) {
                    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(p.gate + (size_t)(t0 + qq_a) * p.gate_stride + h_a * DV + d);
                    x = x / (1.f + __expf(-__low2float(g)));
                    y = y / (1.f + __expf(-__high2float(g)));
                }
                *reinterpret_cast<__nv_bfloat162*>(p.out + (size_t)(t0 + qq_a) * total + h_a * DV + d) = __floats2bfloat162_rn(x, y);
            }
            if (valid_b) {
                float x = o_acc[i][2] * f_b, y = o_acc[i][3] * f_b;
                if (p.gate != nullptr) {
                    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(p.gate + (size_t)(t0 + qq_b) * p.gate_stride + h_b * DV + d);
                    x = x / (1.f + __expf(-__low2float(g)));
                    y = y / (1.f + __expf(-__high2float(g)));
                }
                *reinterpret_cast<__nv_bfloat162*>(p.out + (size_t)(t0 + qq_b) * total + h_b * DV + d) = __floats2bfloat162_rn(x, y);
            }
        }
        return;
    }
    // a piece of the keys: maximum, sum and the unnormalised output go to the scratch
    if (valid_a) {
        const size_t row = (size_t)(t0 + qq_a) * p.splits + split;
        if (quad == 0) { p.part_ml[(row * H + h_a) * 2] = m_a; p.part_ml[(row * H + h_a) * 2 + 1] = l_a; }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i)
            *reinterpret_cast<float2*>(p.part_o + row * total + h_a * DV + i * 8 + 2 * quad) = make_float2(o_acc[i][0], o_acc[i][1]);
    }
    if (valid_b) {
        const size_t row = (size_t)(t0 + qq_b) * p.splits + split;
        if (quad == 0) { p.part_ml[(row * H + h_b) * 2] = m_b; p.part_ml[(row * H + h_b) * 2 + 1] = l_b; }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i)
            *reinterpret_cast<float2*>(p.part_o + row * total + h_b * DV + i * 8 + 2 * quad) = make_float2(o_acc[i][2], o_acc[i][3]);
    }
}

// One block per (token, head): the pieces' maxima, sums and outputs become the row. grid = (tokens, H), DV / 2 threads.
__global__ void attn_mix_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits, int H,
                                        int DV, int sink_one, const bf16* __restrict__ gate, int gate_stride) {
    const int t = blockIdx.x, h = blockIdx.y, total = H * DV, e = h * DV + threadIdx.x * 2;
    const float* ml = part_ml + ((size_t)t * splits * H + h) * 2;
    const float* po = part_o + (size_t)t * splits * total + e;
    float M = sink_one ? 0.f : -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, ml[(size_t)s * H * 2]);
    float L = sink_one ? __expf(-M) : 0.f, x = 0.f, y = 0.f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
        const float m = ml[(size_t)s * H * 2], l = ml[(size_t)s * H * 2 + 1];
        const float2 o = *reinterpret_cast<const float2*>(po + (size_t)s * total);
        const float w = m == -INFINITY ? 0.f : __expf(m - M);
        L = fmaf(l, w, L);
        x = fmaf(o.x, w, x);
        y = fmaf(o.y, w, y);
    }
    const float f = L > 0.f ? 1.f / L : 0.f;
    x *= f;
    y *= f;
    if (gate != nullptr) {
        const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gate + (size_t)t * gate_stride + e);
        x = x / (1.f + __expf(-__low2float(g)));
        y = y / (1.f + __expf(-__high2float(g)));
    }
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * total + e) = __floats2bfloat162_rn(x, y);
}

template <int DK, int DV>
int launch_mix_mma(const MixArgs& a, int n_tiles, size_t smem, cudaStream_t stream) {
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mix_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = smem;
    }
    attn_mix_mma_kernel<DK, DV><<<dim3(n_tiles, a.splits), a.KVH * a.QT * 32, smem, stream>>>(a);
    return oxr_launch_status();
}
}   // namespace

// Shared memory the tiled kernel needs for these sizes with `qt` query parts per block; 0 when it cannot take them at all.
OXR_API long long oxr_attention_mix_mma_smem(int DK, int DV, int H, int KVH, int qt, int single) {
    if ((DK != 64 && DK != 128) || (DV != 64 && DV != 128) || H <= 0 || KVH <= 0 || H % KVH || qt <= 0) return 0;
    const int per = H / KVH;
    if (per > 16 || 16 % per || KVH * qt > MAX_WARPS) return 0;
    return (long long)mix_smem_bytes(DK, DV, H, KVH, (H + 3) & ~3, qt, single ? 1 : qt * (16 / per));
}

// `single`: every tile is one token (a decode step); qt is then 1 and the score exchange keeps one row per head, so two blocks fit an SM.
OXR_API int oxr_attention_mix_mma(void* out, const void* q, int q_stride, const void* k_pool, const void* v_pool, int DK, int DV, int H, int KVH, int qt, int single,
                                  const int* tile_req, const int* tile_tok0, int n_tiles, const int* cu_q, const int* positions, int n_tokens,
                                  const int* block_table, int table_width, int page_size, int num_pages, float scale, float cap, const float* mix,
                                  int sink_one, int window, const void* gate, int gate_stride, int splits, float* part_o, float* part_ml, int* status,
                                  cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return 0;
    const long long smem = oxr_attention_mix_mma_smem(DK, DV, H, KVH, qt, single);
    if ((single && qt != 1) || smem <= 0 || smem > 227 * 1024 || page_size <= 0 || window < 0 || cap < 0.f || splits < 1 || q_stride % 8 || gate_stride % 2 ||
        (splits > 1 && (part_o == nullptr || part_ml == nullptr)))
        return OXR_BAD_ARGUMENT;
    MixArgs a;
    a.out = (bf16*)out; a.q = (const bf16*)q; a.q_stride = q_stride; a.k_pool = (const bf16*)k_pool; a.v_pool = (const bf16*)v_pool;
    a.H = H; a.KVH = KVH; a.HP = (H + 3) & ~3; a.QT = qt; a.SQ = single ? 1 : qt * (16 / (H / KVH));
    a.tile_req = tile_req; a.tile_tok0 = tile_tok0; a.cu_q = cu_q; a.positions = positions;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size; a.num_pages = num_pages;
    a.scale = scale; a.cap = cap; a.mix = mix; a.sink_one = sink_one; a.window = window;
    a.gate = (const bf16*)gate; a.gate_stride = gate_stride; a.splits = splits; a.part_o = part_o; a.part_ml = part_ml; a.status = status;
    int rc;
    if (DK == 64 && DV == 64) rc = launch_mix_mma<64, 64>(a, n_tiles, (size_t)smem, stream);
    else if (DK == 64) rc = launch_mix_mma<64, 128>(a, n_tiles, (size_t)smem, stream);
    else if (DV == 64) rc = launch_mix_mma<128, 64>(a, n_tiles, (size_t)smem, stream);
    else rc = launch_mix_mma<128, 128>(a, n_tiles, (size_t)smem, stream);
    if (rc != 0 || splits == 1) return rc;
    attn_mix_combine_kernel<<<dim3(n_tokens, H), DV / 2, 0, stream>>>((bf16*)out, part_o, part_ml, splits, H, DV, sink_one, (const bf16*)gate, gate_stride);
    return oxr_launch_status();
}
