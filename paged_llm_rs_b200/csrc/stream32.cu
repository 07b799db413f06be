// A residual stream kept in float32 whatever the compute dtype: the kernels of a decoder whose
// residual sum must not be rounded to bfloat16 between layers.
//
//   embed_scaled32      x[t] = table[token[t]] * scale                      (table in T, x in float)
//   sinusoid_add        x[t, 2i] += sin(p_t * f_i),  x[t, 2i+1] += cos(p_t * f_i)   (angle formed in float)
//   round_rows          h = T(x)                                            (what a sublayer's products read)
//   outnorm_add         x[r] += a[r] / sqrt(mean(a[r]^2) + eps) * gain;  h[r] = T(x[r])
//                       (the norm sits on the sublayer's OUTPUT a, the sum stays in float)
//   sandwich_norm32     x[r] += norm(a[r] + bias) * gain_a, then y[i] = T(norm(x[r]) * gain): output norm, sum and input norm
//   rmsnorm_from32      y[i] = T(x[r] / sqrt(mean(x[r]^2) + eps) * gain),  r = rows ? rows[i] : i
//   embed_norm32        x[t] = e / sqrt(mean(e^2) + eps) * gain,  e = table[token[t]]       (a norm right behind the embedding)
//   add_scaled_norm32   x[r] += mult * d[r]  (d may be absent);  y[i] = T(x[r] / sqrt(mean(x[r]^2) + eps) * gain)
//                       (the pre-norm block of a float stream whose sublayer outputs are multiplied by a constant;
//                       with rows the sum is formed for those rows only and not stored)
//   scale32             x *= c
//
// All statistics, the gain multiply and the sum are float; each output is rounded once.
#include "common.cuh"

enum : int { KID_STREAM32 = 40 };

template <typename T>
__global__ void embed_scaled32_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ out,
                                      int hidden, int vocab, float scale, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_f32(src[i]) * scale : 0.f;
}

PLLM_EXPORT int pllm_embed_scaled32(int dtype, const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                                    int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (hidden <= 0 || vocab <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int threads = min(256, max(32, (hidden + 31) / 32 * 32));
        launch_chained(embed_scaled32_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const T*)table, out,
                       hidden, vocab, scale, status);
    });
    return launch_status();
}

// inv_freq holds width / 2 frequencies.  The angle is the float product of the position and the
// frequency; sincosf (the accurate one: this library is not built with fast math) reduces it.
__global__ void sinusoid_add_kernel(float* x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                    int width) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    float* row = x + (size_t)t * width;
    for (int i = threadIdx.x; i < width / 2; i += blockDim.x) {
        float s, c;
        sincosf(p * inv_freq[i], &s, &c);
        float2 v = *reinterpret_cast<float2*>(row + 2 * i);
        v.x += s; v.y += c;
        *reinterpret_cast<float2*>(row + 2 * i) = v;
    }
}

PLLM_EXPORT int pllm_sinusoid_add(float* x, const int* positions, const float* inv_freq, int n_tokens, int width,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (width <= 0 || width % 2) return PLLM_ERR_SIZE;
    const int threads = min(256, max(32, (width / 2 + 31) / 32 * 32));
    launch_chained(sinusoid_add_kernel, dim3(n_tokens), dim3(threads), 0, stream, x, positions, inv_freq, width);
    return launch_status();
}

template <typename T>
__global__ void round_rows_kernel(const float* x, T* __restrict__ h, long long total) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        h[i] = from_f32<T>(x[i]);
}

PLLM_EXPORT int pllm_round_rows(int dtype, const float* x, void* h, long long total, cudaStream_t stream) {
    if (total <= 0) return PLLM_OK;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int blocks = (int)min((long long)sm_count() * 8, (total + 255) / 256);
        launch_chained(round_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, x, (T*)h, total);
    });
    return launch_status();
}

// One row a team of 1 to 8 warps of a 256-thread CTA.  Rows of whole 16-byte vectors of T are read and written as
// vectors (the stream as float4s beside them); the row of `a` is read once for the statistic and once more (from L1)
// for the sum.  h may be null (a float32 engine reads x itself).
template <typename T>
__global__ void __launch_bounds__(256) outnorm_add_kernel(float* x, const T* a, const float* __restrict__ gain, T* h,
                                                          int n_rows, int width, float eps, int team) {
    __shared__ float part[8];
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int r = blockIdx.x * rows_per_cta + warp / team;
    const bool vec = width % N == 0;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = r < n_rows;
    const T* ar = a + (size_t)(live ? r : 0) * width;
    float ss = 0.f;
    if (live) {
        if (vec) {
#pragma unroll 2
            for (int c = member * N; c < width; c += lanes * N) {
                Vec16<T> v; v.load(ar + c);
                float f[N]; v.unpack(f);
#pragma unroll
                for (int k = 0; k < N; k++) ss += f[k] * f[k];
            }
        } else {
            for (int c = member; c < width; c += lanes) { const float v = to_f32(ar[c]); ss += v * v; }
        }
    }
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    float* xr = x + (size_t)r * width;
    T* hr = h ? h + (size_t)r * width : nullptr;
    if (vec) {
#pragma unroll 2
        for (int c = member * N; c < width; c += lanes * N) {
            Vec16<T> v; v.load(ar + c);
            float f[N]; v.unpack(f);
#pragma unroll
            for (int k = 0; k < N; k += 4) {
                float4 s4 = *reinterpret_cast<float4*>(xr + c + k);
                const float4 g4 = *reinterpret_cast<const float4*>(gain + c + k);
                s4.x += f[k] * inv * g4.x; s4.y += f[k + 1] * inv * g4.y; s4.z += f[k + 2] * inv * g4.z; s4.w += f[k + 3] * inv * g4.w;
                *reinterpret_cast<float4*>(xr + c + k) = s4;
                f[k] = s4.x; f[k + 1] = s4.y; f[k + 2] = s4.z; f[k + 3] = s4.w;
            }
            if (hr) { Vec16<T> o; o.pack(f); o.store(hr + c); }
        }
        return;
    }
    for (int c = member; c < width; c += lanes) {
        const float v = xr[c] + to_f32(ar[c]) * inv * gain[c];
        xr[c] = v;
        if (hr) hr[c] = from_f32<T>(v);
    }
}

// warps a row: a lane holds two vectors or so; few rows get more warps each
static inline int stream32_team(int n_rows, int width, int vec) {
    const int per_lane = n_rows <= 64 ? vec : 2 * vec;
    int team = 1;
    while (team < 8 && width > team * 32 * per_lane) team *= 2;
    return team;
}

PLLM_EXPORT int pllm_outnorm_add(int dtype, float* x, const void* a, const float* gain, void* h, int n_rows, int width,
                                 float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int team = stream32_team(n_rows, width, Vec16<T>::N);
        const int rows_per_cta = 8 / team;
        launch_chained(outnorm_add_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       (const T*)a, gain, (T*)h, n_rows, width, eps, team);
    });
    return launch_status();
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_from32_kernel(const float* x, const float* __restrict__ gain, T* __restrict__ y,
                                                             const int* __restrict__ rows, int n_rows, int width, float eps,
                                                             int team) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int i = blockIdx.x * rows_per_cta + warp / team;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = i < n_rows;
    const size_t r = live ? (rows ? (size_t)rows[i] : (size_t)i) : 0;
    const float* xr = x + r * width;
    float ss = 0.f;
    const bool vec = width % 8 == 0;
    if (live) {
        if (vec) {
#pragma unroll 2
            for (int c = member * 4; c < width; c += lanes * 4) {
                const float4 v = *reinterpret_cast<const float4*>(xr + c);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        } else {
            for (int c = member; c < width; c += lanes) { const float v = xr[c]; ss += v * v; }
        }
    }
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* yr = y + (size_t)i * width;
    if (vec) {
        for (int c = member * 4; c < width; c += lanes * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            const float4 g = *reinterpret_cast<const float4*>(gain + c);
            yr[c] = from_f32<T>(v.x * inv * g.x); yr[c + 1] = from_f32<T>(v.y * inv * g.y);
            yr[c + 2] = from_f32<T>(v.z * inv * g.z); yr[c + 3] = from_f32<T>(v.w * inv * g.w);
        }
        return;
    }
    for (int c = member; c < width; c += lanes) yr[c] = from_f32<T>(xr[c] * inv * gain[c]);
}

PLLM_EXPORT int pllm_rmsnorm_from32(int dtype, const float* x, const float* gain, void* y, const int* rows, int n_rows,
                                    int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int team = stream32_team(n_rows, width, 4);
        const int rows_per_cta = 8 / team;
        launch_chained(rmsnorm_from32_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       gain, (T*)y, rows, n_rows, width, eps, team);
    });
    return launch_status();
}

// One CTA a token: the row is fetched once into registers-by-stride, its mean square reduced over the CTA.
template <typename T>
__global__ void __launch_bounds__(256) embed_norm32_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                                           const float* __restrict__ gain, float* __restrict__ out, int hidden,
                                                           int vocab, float eps, int* status) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float v = to_f32(src[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_f32(src[i]) * inv * gain[i] : 0.f;
}

PLLM_EXPORT int pllm_embed_norm32(int dtype, const int* tokens, const void* table, const float* gain, float* out, int n_tokens,
                                  int hidden, int vocab, float eps, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (hidden <= 0 || vocab <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int threads = min(256, max(32, (hidden + 31) / 32 * 32));
        launch_chained(embed_norm32_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const T*)table, gain, out,
                       hidden, vocab, eps, status);
    });
    return launch_status();
}

// Rows and teams as in outnorm_add.  The sum x + mult * d is formed once, kept in registers where the row is short
// enough (ADD_KEEP values a lane) and formed again otherwise; it is stored only when every row is taken (rows null).
#define ADD_KEEP 16
template <typename T>
__global__ void __launch_bounds__(256) add_scaled_norm32_kernel(float* x, const T* d, float mult, const float* __restrict__ gain,
                                                                T* __restrict__ y, const int* __restrict__ rows, int n_rows,
                                                                int width, float eps, int team) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int i = blockIdx.x * rows_per_cta + warp / team;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = i < n_rows;
    const size_t r = live ? (rows ? (size_t)rows[i] : (size_t)i) : 0;
    float* xr = x + r * width;
    const T* dr = d ? d + r * width : nullptr;
    const bool store = d != nullptr && rows == nullptr;
    float keep[ADD_KEEP];
    float ss = 0.f;
    if (live) {
        int k = 0;
        for (int c = member; c < width; c += lanes, k++) {
            float v = xr[c];
            if (dr) v += mult * to_f32(dr[c]);
            if (store) xr[c] = v;
            if (k < ADD_KEEP) keep[k] = v;
            ss += v * v;
        }
    }
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* yr = y + (size_t)i * width;
    int k = 0;
    for (int c = member; c < width; c += lanes, k++) {
        float v;
        if (k < ADD_KEEP) v = keep[k];
        else { v = xr[c]; if (dr && !store) v += mult * to_f32(dr[c]); }
        yr[c] = from_f32<T>(v * inv * gain[c]);
    }
}

PLLM_EXPORT int pllm_add_scaled_norm32(int dtype, float* x, const void* d, float mult, const float* gain, void* y, const int* rows,
                                       int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int team = stream32_team(n_rows, width, 4);
        const int rows_per_cta = 8 / team;
        launch_chained(add_scaled_norm32_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       (const T*)d, mult, gain, (T*)y, rows, n_rows, width, eps, team);
    });
    return launch_status();
}

// A block that norms each sublayer's input AND its output: the output's norm, the sum into the stream and the next
// sublayer's input norm in one pass.  With a' = a + a_bias (a_bias may be null):
//     x[r] += a'[r] / sqrt(mean(a'[r]^2) + eps) * gain_a                     (a given)
//     y[i]  = T(x[r] / sqrt(mean(x[r]^2) + eps) * gain),  r = rows ? rows[i] : i     (y given)
// The sum is stored only when every row is taken (rows null).  Rows and teams as in outnorm_add; a lane keeps up to
// ADD_KEEP values of a row in registers and forms the others again.
template <typename T>
__global__ void __launch_bounds__(256) sandwich_norm32_kernel(float* x, const T* a, const float* __restrict__ a_bias,
                                                              const float* __restrict__ gain_a, const float* __restrict__ gain,
                                                              T* __restrict__ y, const int* __restrict__ rows, int n_rows, int width,
                                                              float eps, int team) {
    __shared__ float part[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int i = blockIdx.x * rows_per_cta + warp / team;
    const int first = warp / team * team;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = i < n_rows;
    const size_t r = live ? (rows ? (size_t)rows[i] : (size_t)i) : 0;
    float* xr = x + r * width;
    const T* ar = a ? a + r * width : nullptr;
    const bool store = a != nullptr && rows == nullptr;
    float keep[ADD_KEEP];
    float inv_a = 0.f;
    if (a != nullptr) {
        float ss = 0.f;
        if (live) {
            int k = 0;
            for (int c = member; c < width; c += lanes, k++) {
                float v = to_f32(ar[c]);
                if (a_bias) v += a_bias[c];
                if (k < ADD_KEEP) keep[k] = v;
                ss += v * v;
            }
        }
        ss = warp_sum(ss);
        if (team > 1) {
            if (lane == 0) part[0][warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int w = 0; w < team; w++) ss += part[0][first + w];
        }
        inv_a = 1.0f / sqrtf(ss / (float)width + eps);
    }
    float ss = 0.f;
    if (live) {
        int k = 0;
        for (int c = member; c < width; c += lanes, k++) {
            float v = xr[c];
            if (ar) {
                float av;
                if (k < ADD_KEEP) av = keep[k];
                else { av = to_f32(ar[c]); if (a_bias) av += a_bias[c]; }
                v += av * inv_a * gain_a[c];
                if (store) xr[c] = v;
            }
            if (k < ADD_KEEP) keep[k] = v;
            ss += v * v;
        }
    }
    if (y == nullptr) return;
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[1][warp] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < team; w++) ss += part[1][first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* yr = y + (size_t)i * width;
    int k = 0;
    for (int c = member; c < width; c += lanes, k++) {
        float v;
        if (k < ADD_KEEP) v = keep[k];
        else {
            v = xr[c];
            if (ar && !store) { float av = to_f32(ar[c]); if (a_bias) av += a_bias[c]; v += av * inv_a * gain_a[c]; }
        }
        yr[c] = from_f32<T>(v * inv * gain[c]);
    }
}

PLLM_EXPORT int pllm_sandwich_norm32(int dtype, float* x, const void* a, const float* a_bias, const float* gain_a, const float* gain,
                                     void* y, const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0 || (a != nullptr && gain_a == nullptr) || (y != nullptr && gain == nullptr)) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int team = stream32_team(n_rows, width, 4);
        const int rows_per_cta = 8 / team;
        launch_chained(sandwich_norm32_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       (const T*)a, a_bias, gain_a, gain, (T*)y, rows, n_rows, width, eps, team);
    });
    return launch_status();
}

// x[r] += mult * d[r] for every row, nothing else (the last sublayer's output when no row is wanted of the step).
template <typename T>
__global__ void add_scaled32_kernel(float* x, const T* d, float mult, long long total) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        x[i] += mult * to_f32(d[i]);
}

PLLM_EXPORT int pllm_add_scaled32(int dtype, float* x, const void* d, float mult, long long total, cudaStream_t stream) {
    if (total <= 0) return PLLM_OK;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int blocks = (int)min((long long)sm_count() * 8, (total + 255) / 256);
        launch_chained(add_scaled32_kernel<T>, dim3(blocks), dim3(256), 0, stream, x, (const T*)d, mult, total);
    });
    return launch_status();
}

__global__ void scale32_kernel(float* x, float c, long long total) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) x[i] *= c;
}

PLLM_EXPORT int pllm_scale32(float* x, float c, long long total, cudaStream_t stream) {
    if (total <= 0) return PLLM_OK;
    const int blocks = (int)min((long long)sm_count() * 8, (total + 255) / 256);
    launch_chained(scale32_kernel, dim3(blocks), dim3(256), 0, stream, x, c, total);
    return launch_status();
}

PLLM_TRACE_EXPORT(stream32)
