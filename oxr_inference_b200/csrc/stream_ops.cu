// Operations on a residual stream that is kept whole in fp32: RMSNorm of the stream, the post-norm add
// (stream += norm(y) * w, optionally followed by the next pre-norm in the same pass), the concatenation that feeds a
// re-entry map, a broadcast row add, a gated feed-forward activation with clamps, and per-step rotary angles.
//
// All arithmetic is fp32 (the angles: fp64, rounded once); T is the activation type that the products read and write.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------- norm of the stream
// One block per output row; row r reads stream row `rows ? rows[r] : r`. out = x * rsqrt(mean(x^2) + eps) * weight.
template <typename T>
__global__ void stream_rms_norm_kernel(T* __restrict__ out, const float* __restrict__ stream, const float* __restrict__ weight,
                                       const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* x = stream + (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)hidden + eps);
    T* dst = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Num<T>::from_f32(x[i] * inv * weight[i]);
}

// stream[r] += y[r] * rsqrt(mean(y[r]^2) + eps) * w_post; then, when `out` is given, out[r] = norm(stream[r]) * w_next.
// One block per row; the updated row is kept in shared memory for the second norm when it fits.
template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ stream, const T* __restrict__ y, const float* __restrict__ w_post,
                                     T* __restrict__ out, const float* __restrict__ w_next, int hidden, float eps_post, float eps_next,
                                     int row_floats_in_smem) {
    extern __shared__ float smem[];
    float* red = smem;
    float* rowbuf = smem + 32;
    const size_t at = (size_t)blockIdx.x * hidden;
    const bool cached = row_floats_in_smem >= hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = Num<T>::to_f32(y[at + i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)hidden + eps_post);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = stream[at + i] + Num<T>::to_f32(y[at + i]) * inv * w_post[i];
        stream[at + i] = v;
        if (cached) rowbuf[i] = v;
        s2 = fmaf(v, v, s2);
    }
    if (out == nullptr) return;
    if (w_next == nullptr) {   // no norm behind the add: the new stream, rounded
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[at + i] = Num<T>::from_f32(cached ? rowbuf[i] : stream[at + i]);
        return;
    }
    s2 = block_sum(s2, red);
    const float inv2 = 1.f / sqrtf(s2 / (float)hidden + eps_next);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = cached ? rowbuf[i] : stream[at + i];   // written by this same thread above
        out[at + i] = Num<T>::from_f32(v * inv2 * w_next[i]);
    }
}

// The same for bf16 rows that are whole 16-byte words: a thread keeps its VPT words of y and of the stream in registers from the
// first load to the last store, so every row is read once, with 16-byte loads.
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&out)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&v)[8]) {
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return out;
}

template <int VPT>
__global__ void norm_add_norm_bf16x8_kernel(float* __restrict__ stream, const __nv_bfloat16* __restrict__ y, const float* __restrict__ w_post,
                                            __nv_bfloat16* __restrict__ out, const float* __restrict__ w_next, int hidden, float eps_post,
                                            float eps_next) {
    __shared__ float red[32];
    const size_t at = (size_t)blockIdx.x * hidden;
    const int nvec = hidden / 8;
    float yv[VPT][8], sv[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * blockDim.x;
        if (idx < nvec) {
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(y + at + 8 * idx), yv[v]);
            const float4 a = *reinterpret_cast<const float4*>(stream + at + 8 * idx), b = *reinterpret_cast<const float4*>(stream + at + 8 * idx + 4);
            sv[v][0] = a.x; sv[v][1] = a.y; sv[v][2] = a.z; sv[v][3] = a.w; sv[v][4] = b.x; sv[v][5] = b.y; sv[v][6] = b.z; sv[v][7] = b.w;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(yv[v][i], yv[v][i], ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)hidden + eps_post);
    float s2 = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * blockDim.x;
        if (idx < nvec) {
            const float4 wa = *reinterpret_cast<const float4*>(w_post + 8 * idx), wb = *reinterpret_cast<const float4*>(w_post + 8 * idx + 4);
            const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sv[v][i] += yv[v][i] * inv * w[i];
                s2 = fmaf(sv[v][i], sv[v][i], s2);
            }
            *reinterpret_cast<float4*>(stream + at + 8 * idx) = make_float4(sv[v][0], sv[v][1], sv[v][2], sv[v][3]);
            *reinterpret_cast<float4*>(stream + at + 8 * idx + 4) = make_float4(sv[v][4], sv[v][5], sv[v][6], sv[v][7]);
        }
    }
    if (out == nullptr) return;
    if (w_next == nullptr) {   // no norm behind the add: the new stream, rounded
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int idx = threadIdx.x + v * blockDim.x;
            if (idx < nvec) *reinterpret_cast<uint4*>(out + at + 8 * idx) = f32_to_bf16x8(sv[v]);
        }
        return;
    }
    s2 = block_sum(s2, red);
    const float inv2 = 1.f / sqrtf(s2 / (float)hidden + eps_next);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * blockDim.x;
        if (idx < nvec) {
            const float4 wa = *reinterpret_cast<const float4*>(w_next + 8 * idx), wb = *reinterpret_cast<const float4*>(w_next + 8 * idx + 4);
            const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = sv[v][i] * inv2 * w[i];
            *reinterpret_cast<uint4*>(out + at + 8 * idx) = f32_to_bf16x8(o);
        }
    }
}

// out[r] = [ a[r] | b[r] ] rounded to T
template <typename T>
__global__ void concat2_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b, int hidden, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (2 * hidden);
        const int c = (int)(i % (2 * hidden));
        out[i] = Num<T>::from_f32(c < hidden ? a[r * hidden + c] : b[r * hidden + (c - hidden)]);
    }
}

__global__ void add_row_f32_kernel(float* __restrict__ x, const float* __restrict__ row, int hidden, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] += row[i % hidden];
}

// ---------------------------------------------------------------------------------------------- clamped gated unit
// out = g' * sigmoid(alpha * g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit); gate_up rows are
// [gate | up] (interleave 0) or gate and up alternating in groups of `interleave` columns.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, int interleave, float alpha, float limit,
                                   size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / inter;
        const int col = (int)(i % inter);
        size_t gi, ui;
        if (interleave) {
            gi = row * 2 * inter + (size_t)(col / interleave) * 2 * interleave + col % interleave;
            ui = gi + interleave;
        } else {
            gi = row * 2 * inter + col;
            ui = gi + inter;
        }
        const float g = fminf(Num<T>::to_f32(gate_up[gi]), limit);
        const float u = fminf(fmaxf(Num<T>::to_f32(gate_up[ui]), -limit), limit);
        out[i] = Num<T>::from_f32(g / (1.f + expf(-alpha * g)) * (u + 1.f));
    }
}

// bf16, [gate | up] side by side, `inter` a multiple of 8: 16-byte loads and stores. Grid (column words, rows).
__global__ void clamped_glu_bf16x8_kernel(uint4* __restrict__ out, const uint4* __restrict__ gate_up, int inter8, float alpha, float limit) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= inter8) return;
    const size_t row = blockIdx.y;
    float g[8], u[8], o[8];
    bf16x8_to_f32(gate_up[row * 2 * inter8 + c], g);
    bf16x8_to_f32(gate_up[row * 2 * inter8 + inter8 + c], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float gg = fminf(g[i], limit), uu = fminf(fmaxf(u[i], -limit), limit);
        o[i] = gg / (1.f + __expf(-alpha * gg)) * (uu + 1.f);
    }
    out[row * inter8 + c] = f32_to_bf16x8(o);
}

// ---------------------------------------------------------------------------------------------- rotary angles
// cos/sin [tokens, half] of position * freq[i], the product and the functions in fp64, rounded once to fp32.
__global__ void rotary_angles_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out, const int* __restrict__ positions,
                                     const double* __restrict__ freq, int half, int total) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    double s, c;
    sincos((double)positions[i / half] * freq[i % half], &s, &c);
    cos_out[i] = (float)c;
    sin_out[i] = (float)s;
}

// ---------------------------------------------------------------------------------------------- launchers
static inline int grid_for(size_t total, int threads) {
    size_t b = (total + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

OXR_API int oxr_stream_rms_norm(void* out, const float* stream, const float* weight, const int* rows, int n_out, int hidden, float eps,
                                int dtype, cudaStream_t stream_) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == 0) stream_rms_norm_kernel<float><<<n_out, threads, 0, stream_>>>((float*)out, stream, weight, rows, hidden, eps);
    else stream_rms_norm_kernel<__nv_bfloat16><<<n_out, threads, 0, stream_>>>((__nv_bfloat16*)out, stream, weight, rows, hidden, eps);
    return oxr_launch_status();
}

OXR_API int oxr_norm_add_norm(float* stream, const void* y, const float* w_post, void* out, const float* w_next, int n, int hidden,
                              float eps_post, float eps_next, int dtype, cudaStream_t stream_) {
    if (n <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    if (dtype == 1 && hidden % 8 == 0 && hidden <= 32768 && (uintptr_t)stream % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 &&
        (uintptr_t)w_post % 16 == 0 && (uintptr_t)w_next % 16 == 0) {
        const int nvec = hidden / 8;
        const int vpt = nvec <= 512 ? 1 : (nvec <= 2048 ? 2 : 4);
        const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
        const __nv_bfloat16* yb = (const __nv_bfloat16*)y;
        __nv_bfloat16* ob = (__nv_bfloat16*)out;
        if (vpt == 1) norm_add_norm_bf16x8_kernel<1><<<n, threads, 0, stream_>>>(stream, yb, w_post, ob, w_next, hidden, eps_post, eps_next);
        else if (vpt == 2) norm_add_norm_bf16x8_kernel<2><<<n, threads, 0, stream_>>>(stream, yb, w_post, ob, w_next, hidden, eps_post, eps_next);
        else norm_add_norm_bf16x8_kernel<4><<<n, threads, 0, stream_>>>(stream, yb, w_post, ob, w_next, hidden, eps_post, eps_next);
        return oxr_launch_status();
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    const int keep = hidden <= 8192 ? hidden : 0;
    const size_t smem = (32 + keep) * sizeof(float);
    if (dtype == 0)
        norm_add_norm_kernel<float><<<n, threads, smem, stream_>>>(stream, (const float*)y, w_post, (float*)out, w_next, hidden, eps_post, eps_next, keep);
    else
        norm_add_norm_kernel<__nv_bfloat16><<<n, threads, smem, stream_>>>(stream, (const __nv_bfloat16*)y, w_post, (__nv_bfloat16*)out, w_next, hidden,
                                                                          eps_post, eps_next, keep);
    return oxr_launch_status();
}

OXR_API int oxr_concat2_cast(void* out, const float* a, const float* b, int n, int hidden, int dtype, cudaStream_t stream_) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * 2 * hidden;
    if (dtype == 0) concat2_cast_kernel<float><<<grid_for(total, 256), 256, 0, stream_>>>((float*)out, a, b, hidden, total);
    else concat2_cast_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream_>>>((__nv_bfloat16*)out, a, b, hidden, total);
    return oxr_launch_status();
}

OXR_API int oxr_add_row_f32(float* x, const float* row, int n, int hidden, cudaStream_t stream_) {
    if (n <= 0) return 0;
    const size_t total = (size_t)n * hidden;
    add_row_f32_kernel<<<grid_for(total, 256), 256, 0, stream_>>>(x, row, hidden, total);
    return oxr_launch_status();
}

OXR_API int oxr_clamped_glu(void* out, const void* gate_up, int n, int inter, int interleave, float alpha, float limit, int dtype,
                            cudaStream_t stream_) {
    if (n <= 0) return 0;
    if (inter <= 0 || interleave < 0 || (interleave && inter % interleave)) return OXR_BAD_ARGUMENT;
    if (dtype == 1 && interleave == 0 && inter % 8 == 0 && n <= 65535 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0) {
        dim3 grid((inter / 8 + 127) / 128, n);
        clamped_glu_bf16x8_kernel<<<grid, 128, 0, stream_>>>((uint4*)out, (const uint4*)gate_up, inter / 8, alpha, limit);
        return oxr_launch_status();
    }
    const size_t total = (size_t)n * inter;
    if (dtype == 0) clamped_glu_kernel<float><<<grid_for(total, 256), 256, 0, stream_>>>((float*)out, (const float*)gate_up, inter, interleave, alpha, limit, total);
    else clamped_glu_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream_>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter, interleave,
                                                                                     alpha, limit, total);
    return oxr_launch_status();
}

OXR_API int oxr_rotary_angles(float* cos_out, float* sin_out, const int* positions, const double* freq, int n, int half, cudaStream_t stream_) {
    if (n <= 0 || half <= 0) return 0;
    const int total = n * half;
    rotary_angles_kernel<<<(total + 127) / 128, 128, 0, stream_>>>(cos_out, sin_out, positions, freq, half, total);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- layer norm of the stream
// out[r] = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight + bias for stream row `rows ? rows[r] : r`; the mean first,
// then the mean of the squared deviations (two passes, not E[x^2] - E[x]^2), all in fp32. One block per output row.
// The row is read once into shared memory (dynamic: hidden floats); the three passes run there. Rows of a multiple of four entries
// move as 16-byte pieces.
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
}

template <typename T>
__device__ __forceinline__ void layer_norm_of_row(T* __restrict__ dst, const float* row, float sum, const float* __restrict__ weight,
                                                  const float* __restrict__ bias, int hidden, float eps, float* red) {
    const float mean = block_sum(sum, red) / (float)hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    if ((hidden & 3) == 0) {
        for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
            const float4 x = reinterpret_cast<const float4*>(row)[i], w = reinterpret_cast<const float4*>(weight)[i];
            const float4 b = bias != nullptr ? reinterpret_cast<const float4*>(bias)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            store4(dst + 4 * i, make_float4((x.x - mean) * inv * w.x + b.x, (x.y - mean) * inv * w.y + b.y, (x.z - mean) * inv * w.z + b.z,
                                            (x.w - mean) * inv * w.w + b.w));
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float b = bias != nullptr ? bias[i] : 0.f;
        dst[i] = Num<T>::from_f32((row[i] - mean) * inv * weight[i] + b);
    }
}

// The norm's weight and bias are wanted only after two block-wide sums: asked for early, they are in L2 by then.
__device__ __forceinline__ void prefetch_row(const float* p, int hidden) {
    if (p == nullptr) return;
    for (int i = threadIdx.x * 32; i < hidden; i += blockDim.x * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + i));
}

template <typename T>
__global__ void stream_layer_norm_kernel(T* __restrict__ out, const float* __restrict__ stream, const float* __restrict__ weight,
                                         const float* __restrict__ bias, const int* __restrict__ rows, int hidden, float eps) {
    extern __shared__ __align__(16) float ln_row[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* x = stream + (size_t)(rows ? rows[r] : r) * hidden;
    prefetch_row(weight, hidden);
    prefetch_row(bias, hidden);
    float s = 0.f;
    if ((hidden & 3) == 0) {
#pragma unroll 4
        for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(x)[i];
            reinterpret_cast<float4*>(ln_row)[i] = v;
            s += (v.x + v.y) + (v.z + v.w);
        }
    } else {
#pragma unroll 4
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = x[i];
            ln_row[i] = v;
            s += v;
        }
    }
    layer_norm_of_row<T>(out + (size_t)r * hidden, ln_row, s, weight, bias, hidden, eps, red);
}

template <typename K>
static int with_row_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    if (bytes > 200 * 1024) return OXR_BAD_ARGUMENT;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? 0 : 1000 + (int)e;
}

OXR_API int oxr_stream_layer_norm(void* out, const float* stream, const float* weight, const float* bias, const int* rows, int n_out, int hidden,
                                  float eps, int dtype, cudaStream_t stream_) {
    if (n_out <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    const int threads = hidden >= 1024 ? 256 : 128;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (dtype == 0) {
        if (int rc = with_row_smem(stream_layer_norm_kernel<float>, smem)) return rc;
        stream_layer_norm_kernel<float><<<n_out, threads, smem, stream_>>>((float*)out, stream, weight, bias, rows, hidden, eps);
    } else {
        if (int rc = with_row_smem(stream_layer_norm_kernel<__nv_bfloat16>, smem)) return rc;
        stream_layer_norm_kernel<__nv_bfloat16><<<n_out, threads, smem, stream_>>>((__nv_bfloat16*)out, stream, weight, bias, rows, hidden, eps);
    }
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- gated residual, depth average
// What a block with side-by-side sublayers does to the fp32 stream once both sublayers are done, in one pass:
//
//   X = stream + ( a * sigmoid(ga + ba) + f * sigmoid(gf + bf) )          the gates (ga, gf: columns 0.. and hidden.. of `gates`, with
//                                                                        fp32 biases) are optional, and so is the second sublayer f;
//   history[index] = X                                                   when a history [slots, tokens, hidden] is kept, and then
//   stream = sum_{j < index} mixw[j] * history[j] + mixw[index] * X       (the sum in the order of j), else stream = X.
//
// ab / fb: an optional fp32 bias row added to a / f before anything else (a sublayer's output bias).
// What the sublayers add at place i = (row, c): the gated sum y, read-only.
template <typename T>
__device__ __forceinline__ float gated_sum_at(size_t i, size_t row, int c, const T* __restrict__ a, const float* __restrict__ ab,
                                              const T* __restrict__ f, const float* __restrict__ fb, const T* __restrict__ gates, int gates_stride,
                                              const float* __restrict__ gate_bias, int hidden) {
    float y = Num<T>::to_f32(a[i]);
    if (ab != nullptr) y += ab[c];
    if (gates != nullptr) {
        const float g = Num<T>::to_f32(gates[row * gates_stride + c]) + (gate_bias != nullptr ? gate_bias[c] : 0.f);
        y = y / (1.f + expf(-g));
    }
    if (f != nullptr) {
        float z = Num<T>::to_f32(f[i]);
        if (fb != nullptr) z += fb[c];
        if (gates != nullptr) {
            const float g = Num<T>::to_f32(gates[row * gates_stride + hidden + c]) + (gate_bias != nullptr ? gate_bias[hidden + c] : 0.f);
            z = z / (1.f + expf(-g));
        }
        y += z;
    }
    return y;
}

// A load that the compiler knows to be from global memory: it need not wait for the stores to shared memory before it.
__device__ __forceinline__ float global_f32(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// sum_{j < index} mixw[j] * history[j][i], added in the order of j; eight loads are asked for before the first is used
__device__ __forceinline__ float history_sum(const float* history, const float* __restrict__ mixw, int index, size_t total, size_t i) {
    float acc = 0.f;
    for (int j0 = 0; j0 < index; j0 += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = j0 + u < index ? global_f32(history + (size_t)(j0 + u) * total + i) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (j0 + u < index) acc = fmaf(mixw[j0 + u], v[u], acc);
    }
    return acc;
}

template <typename T>
__global__ void gated_residual_kernel(float* __restrict__ stream, const T* __restrict__ a, const float* __restrict__ ab, const T* __restrict__ f,
                                      const float* __restrict__ fb, const T* __restrict__ gates, int gates_stride, const float* __restrict__ gate_bias,
                                      float* __restrict__ history, int index, const float* __restrict__ mixw, int hidden, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / hidden;
        float x = stream[i] + gated_sum_at<T>(i, row, (int)(i - row * hidden), a, ab, f, fb, gates, gates_stride, gate_bias, hidden);
        if (history != nullptr) {
            history[(size_t)index * total + i] = x;
            float acc = 0.f;
            for (int j = 0; j < index; ++j) acc = fmaf(mixw[j], history[(size_t)j * total + i], acc);
            x = fmaf(mixw[index], x, acc);
        }
        stream[i] = x;
    }
}

// The same, one block per row, and the row goes on through the layer norm that reads it next (weight, bias, eps): out = LN(new stream row).
// Two passes: the first only reads global memory (the new row X and the weighted sum go to shared memory), so that its loads run ahead
// of each other; the second writes X to the history and the sum to the stream. Shared memory: 2 * hidden floats.
template <typename T>
__global__ void gated_residual_norm_kernel(T* __restrict__ out, float* stream, const T* __restrict__ a, const float* __restrict__ ab,
                                           const T* __restrict__ f, const float* __restrict__ fb, const T* __restrict__ gates, int gates_stride,
                                           const float* __restrict__ gate_bias, float* history, int index, const float* __restrict__ mixw,
                                           int hidden, size_t total, const float* __restrict__ weight, const float* __restrict__ bias, float eps) {
    extern __shared__ __align__(16) float ln_row[];   // [hidden] the stream's new row, then [hidden] X
    __shared__ float red[32];
    float* x_row = ln_row + hidden;
    const size_t row = blockIdx.x;
    prefetch_row(weight, hidden);
    prefetch_row(bias, hidden);
    float s = 0.f;
#pragma unroll 2
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const size_t i = row * hidden + c;
        float x = global_f32(stream + i) + gated_sum_at<T>(i, row, c, a, ab, f, fb, gates, gates_stride, gate_bias, hidden);
        x_row[c] = x;
        if (history != nullptr) {
            x = fmaf(mixw[index], x, history_sum(history, mixw, index, total, i));
        }
        ln_row[c] = x;
        s += x;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const size_t i = row * hidden + c;
        if (history != nullptr) history[(size_t)index * total + i] = x_row[c];
        stream[i] = ln_row[c];
    }
    layer_norm_of_row<T>(out + row * hidden, ln_row, s, weight, bias, hidden, eps, red);
}

OXR_API int oxr_gated_residual_norm(void* out, float* stream, const void* a, const float* ab, const void* f, const float* fb, const void* gates,
                                    int gates_stride, const float* gate_bias, float* history, int index, const float* mixw, int n, int hidden,
                                    const float* weight, const float* bias, float eps, int dtype, cudaStream_t stream_) {
    if (n <= 0) return 0;
    if (hidden <= 0 || a == nullptr || weight == nullptr || (history != nullptr && (mixw == nullptr || index < 0))) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n * hidden, smem = 2 * (size_t)hidden * sizeof(float);
    const int threads = hidden >= 4096 ? 1024 : hidden >= 2048 ? 512 : hidden >= 1024 ? 256 : 128;   // every thread's loads of a row are in flight together
    if (dtype == 0) {
        if (int rc = with_row_smem(gated_residual_norm_kernel<float>, smem)) return rc;
        gated_residual_norm_kernel<float><<<n, threads, smem, stream_>>>((float*)out, stream, (const float*)a, ab, (const float*)f, fb, (const float*)gates,
                                                                        gates_stride, gate_bias, history, index, mixw, hidden, total, weight, bias, eps);
    } else {
        typedef __nv_bfloat16 B;
        if (int rc = with_row_smem(gated_residual_norm_kernel<B>, smem)) return rc;
        gated_residual_norm_kernel<B><<<n, threads, smem, stream_>>>((B*)out, stream, (const B*)a, ab, (const B*)f, fb, (const B*)gates, gates_stride,
                                                                    gate_bias, history, index, mixw, hidden, total, weight, bias, eps);
    }
    return oxr_launch_status();
}

OXR_API int oxr_gated_residual(float* stream, const void* a, const float* ab, const void* f, const float* fb, const void* gates, int gates_stride,
                               const float* gate_bias, float* history, int index, const float* mixw, int n, int hidden, int dtype,
                               cudaStream_t stream_) {
    if (n <= 0) return 0;
    if (hidden <= 0 || a == nullptr || (history != nullptr && (mixw == nullptr || index < 0))) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n * hidden;
    if (dtype == 0)
        gated_residual_kernel<float><<<grid_for(total, 256), 256, 0, stream_>>>(stream, (const float*)a, ab, (const float*)f, fb, (const float*)gates,
                                                                               gates_stride, gate_bias, history, index, mixw, hidden, total);
    else
        gated_residual_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream_>>>(stream, (const __nv_bfloat16*)a, ab, (const __nv_bfloat16*)f, fb,
                                                                                       (const __nv_bfloat16*)gates, gates_stride, gate_bias, history,
                                                                                       index, mixw, hidden, total);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- tanh GELU
// out = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), fp32 arithmetic, rounded once; out may be x itself.
template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ out, const T* __restrict__ x, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float z = Num<T>::to_f32(x[i]);
        out[i] = Num<T>::from_f32(0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))));
    }
}

__global__ void gelu_tanh_bf16x8_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, size_t total8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        float z[8], o[8];
        bf16x8_to_f32(x[i], z);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = 0.5f * z[k] * (1.f + tanhf(0.7978845608028654f * (z[k] + 0.044715f * z[k] * z[k] * z[k])));
        out[i] = f32_to_bf16x8(o);
    }
}

OXR_API int oxr_gelu_tanh(void* out, const void* x, long long total, int dtype, cudaStream_t stream_) {
    if (total <= 0) return 0;
    if (dtype == 1 && total % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0) {
        gelu_tanh_bf16x8_kernel<<<grid_for((size_t)total / 8, 256), 256, 0, stream_>>>((uint4*)out, (const uint4*)x, (size_t)total / 8);
        return oxr_launch_status();
    }
    if (dtype == 0) gelu_tanh_kernel<float><<<grid_for((size_t)total, 256), 256, 0, stream_>>>((float*)out, (const float*)x, (size_t)total);
    else gelu_tanh_kernel<__nv_bfloat16><<<grid_for((size_t)total, 256), 256, 0, stream_>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (size_t)total);
    return oxr_launch_status();
}

// y += x element by element (the sum in fp32, rounded once)
template <typename T>
__global__ void add_inplace_kernel(T* __restrict__ y, const T* __restrict__ x, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] = Num<T>::from_f32(Num<T>::to_f32(y[i]) + Num<T>::to_f32(x[i]));
}

OXR_API int oxr_add_inplace(void* y, const void* x, long long total, int dtype, cudaStream_t stream_) {
    if (total <= 0) return 0;
    if (dtype == 0) add_inplace_kernel<float><<<grid_for((size_t)total, 256), 256, 0, stream_>>>((float*)y, (const float*)x, (size_t)total);
    else add_inplace_kernel<__nv_bfloat16><<<grid_for((size_t)total, 256), 256, 0, stream_>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)x, (size_t)total);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- two mixers side by side
// out[r] = 0.5 * (a[r] / rms(a[r]) * wa + b[r] / rms(b[r]) * wb): the mean of two results, each RMS-normed over the row with a weight of
// its own; sums of squares, norms and the mean in fp32, rounded once. One block per row.
template <typename T>
__global__ void pair_norm_mean_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                                      const float* __restrict__ wb, int hidden, float eps) {
    __shared__ float red[32];
    const size_t at = (size_t)blockIdx.x * hidden;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float x = Num<T>::to_f32(a[at + i]), y = Num<T>::to_f32(b[at + i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    sa = block_sum(sa, red);
    sb = block_sum(sb, red);
    const float ia = 1.f / sqrtf(sa / (float)hidden + eps), ib = 1.f / sqrtf(sb / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[at + i] = Num<T>::from_f32(0.5f * (Num<T>::to_f32(a[at + i]) * ia * wa[i] + Num<T>::to_f32(b[at + i]) * ib * wb[i]));
}

// The same for bf16 rows that are whole 16-byte words: a thread keeps its VPT words of both inputs in registers, so every row is read once.
template <int VPT>
__global__ void pair_norm_mean_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                             const float* __restrict__ wa, const float* __restrict__ wb, int hidden, float eps) {
    __shared__ float red[32];
    const size_t at = (size_t)blockIdx.x * hidden;
    const int nvec = hidden / 8;
    float av[VPT][8], bv[VPT][8];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * blockDim.x;
        if (idx < nvec) {
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(a + at + 8 * idx), av[v]);
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(b + at + 8 * idx), bv[v]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sa = fmaf(av[v][i], av[v][i], sa);
                sb = fmaf(bv[v][i], bv[v][i], sb);
            }
        }
    }
    sa = block_sum(sa, red);
    sb = block_sum(sb, red);
    const float ia = 0.5f / sqrtf(sa / (float)hidden + eps), ib = 0.5f / sqrtf(sb / (float)hidden + eps);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * blockDim.x;
        if (idx < nvec) {
            const float4 a0 = *reinterpret_cast<const float4*>(wa + 8 * idx), a1 = *reinterpret_cast<const float4*>(wa + 8 * idx + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(wb + 8 * idx), b1 = *reinterpret_cast<const float4*>(wb + 8 * idx + 4);
            const float wva[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, wvb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = av[v][i] * ia * wva[i] + bv[v][i] * ib * wvb[i];
            *reinterpret_cast<uint4*>(out + at + 8 * idx) = f32_to_bf16x8(o);
        }
    }
}

OXR_API int oxr_pair_norm_mean(void* out, const void* a, const void* b, const float* wa, const float* wb, int n, int hidden, float eps, int dtype,
                               cudaStream_t stream_) {
    if (n <= 0) return 0;
    if (hidden <= 0) return OXR_BAD_ARGUMENT;
    if (dtype == 1 && hidden % 8 == 0 && hidden <= 32768 && (uintptr_t)out % 16 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 &&
        (uintptr_t)wa % 16 == 0 && (uintptr_t)wb % 16 == 0) {
        const int nvec = hidden / 8;
        const int vpt = nvec <= 512 ? 1 : (nvec <= 2048 ? 2 : 4);
        const int threads_v = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
        const __nv_bfloat16 *ab = (const __nv_bfloat16*)a, *bb = (const __nv_bfloat16*)b;
        if (vpt == 1) pair_norm_mean_bf16x8_kernel<1><<<n, threads_v, 0, stream_>>>((__nv_bfloat16*)out, ab, bb, wa, wb, hidden, eps);
        else if (vpt == 2) pair_norm_mean_bf16x8_kernel<2><<<n, threads_v, 0, stream_>>>((__nv_bfloat16*)out, ab, bb, wa, wb, hidden, eps);
        else pair_norm_mean_bf16x8_kernel<4><<<n, threads_v, 0, stream_>>>((__nv_bfloat16*)out, ab, bb, wa, wb, hidden, eps);
        return oxr_launch_status();
    }
    const int threads = hidden >= 2048 ? 256 : 128;
    if (dtype == 0) pair_norm_mean_kernel<float><<<n, threads, 0, stream_>>>((float*)out, (const float*)a, (const float*)b, wa, wb, hidden, eps);
    else pair_norm_mean_kernel<__nv_bfloat16><<<n, threads, 0, stream_>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, wa, wb, hidden, eps);
    return oxr_launch_status();
}

// x <- cap * tanh(x / cap), fp32, in place (capped logits).
__global__ void tanh_cap_kernel(float* __restrict__ x, float cap, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] = cap * tanhf(x[i] / cap);
}

OXR_API int oxr_tanh_cap(float* x, float cap, long long total, cudaStream_t stream_) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return OXR_BAD_ARGUMENT;
    tanh_cap_kernel<<<grid_for((size_t)total, 256), 256, 0, stream_>>>(x, cap, (size_t)total);
    return oxr_launch_status();
}
