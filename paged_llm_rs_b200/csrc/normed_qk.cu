// What stands between an attention mixer's input projection and its attention kernel, for mixers that norm their
// queries and keys, and the gate on an attention's output.
//
//   normed_qk_kv_write   one pass over the stacked projection [q | k | (v) | ...] of the step's tokens, a CTA a token:
//                          norm      0 none; 1 each head by its own root mean square, one gain of dk entries shared by the
//                                    heads; 2 the whole projection (all heads of q, and likewise of k) by one root mean
//                                    square, a gain of its full size
//                          q *= 1 + coef * ln(floor((p + 1) / every) + 1)     (every = 0: no such factor)
//                          rotation of the first `rot` entries of every q and k head, entry i with entry i + rot / 2, by the
//                                    angle p * inv_freq[i], a float product
//                          q to its own tensor; k | v to the token's row of the joined pool; v is the projection's v
//                          part, or (values_are_keys) the raw key projection, neither normed nor rotated
//                        Everything is float from the projection's values to the one rounding on the way out.
//   gate_mul             y[t, c] *= sigmoid(g[t, c / per]) (kind 0) or silu(g[t, c / per]) (kind 1); g rows may be strided; per 1: a
//                        gate an entry, per = a head's size: a gate a head
#include "common.cuh"

enum : int { KID_NORMED_QK = 90 };

__device__ __forceinline__ float nq_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// Sum over the CTA, for every thread (scratch: 32 floats).
__device__ __forceinline__ float nq_block_sum(float v, float* scratch) { return block_sum(v, scratch); }

template <typename T>
__global__ void __launch_bounds__(256) normed_qk_kv_write_kernel(const T* proj, int row_stride, int k_off, int v_off, T* __restrict__ q_out,
                                                                 const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                                                 int norm, float eps, float temp_coef, int temp_every,
                                                                 const float* __restrict__ inv_freq, int rot,
                                                                 const int* __restrict__ positions, const int* __restrict__ slots,
                                                                 T* kv_pool, int nh, int nkv, int dk, int dv, int values_are_keys,
                                                                 int page_size, long long pool_rows, int* status) {
    extern __shared__ float nq_smem[];
    float* head_inv = nq_smem;            // [nh + nkv] 1 / rms of each head (norm 1)
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait(KID_NORMED_QK);
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * row_stride;
    const T* kr = row + k_off;
    const int pos = positions[t];
    const float p = (float)pos;
    const int half = rot / 2;
    const int qw = nh * dk, kw = nkv * dk;
    float q_inv = 1.f, k_inv = 1.f;
    if (norm == 2) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < qw; i += blockDim.x) { const float v = to_f32(row[i]); sq += v * v; }
        for (int i = threadIdx.x; i < kw; i += blockDim.x) { const float v = to_f32(kr[i]); sk += v * v; }
        sq = nq_block_sum(sq, scratch);
        sk = nq_block_sum(sk, scratch);
        q_inv = 1.0f / sqrtf(sq / (float)qw + eps);
        k_inv = 1.0f / sqrtf(sk / (float)kw + eps);
    } else if (norm == 1) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
        for (int h = warp; h < nh + nkv; h += warps) {
            const T* hr = h < nh ? row + (size_t)h * dk : kr + (size_t)(h - nh) * dk;
            float s = 0.f;
            for (int e = lane; e < dk; e += 32) { const float v = to_f32(hr[e]); s += v * v; }
            s = warp_sum(s);
            if (lane == 0) head_inv[h] = 1.0f / sqrtf(s / (float)dk + eps);
        }
        __syncthreads();
    }
    float temp = 1.f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    // queries
    T* qo = q_out + (size_t)t * qw;
    for (int i = threadIdx.x; i < qw; i += blockDim.x) {
        const int h = i / dk, e = i % dk;
        const float inv = norm == 2 ? q_inv : norm == 1 ? head_inv[h] : 1.f;
        float v = to_f32(row[i]) * inv;
        if (norm) v *= q_gain[norm == 2 ? i : e];
        if (e < rot) {
            const int f = e < half ? e : e - half;
            const int j = e < half ? i + half : i - half;
            float s, c;
            sincosf(p * inv_freq[f], &s, &c);
            float other = to_f32(row[j]) * inv;
            if (norm) other *= q_gain[norm == 2 ? j : (e < half ? e + half : e - half)];
            v = e < half ? v * c - other * s : v * c + other * s;
        }
        qo[i] = from_f32<T>(v * temp);
    }
    const int slot = slots ? slots[t] : -1;
    if (kv_pool == nullptr || slot < 0) return;
    if ((long long)slot >= pool_rows) { if (threadIdx.x == 0) atomicOr(status, 2); return; }
    const int page = slot / page_size, off = slot % page_size;
    const int w = dk + dv;
    const T* vr = row + v_off;
    for (int i = threadIdx.x; i < nkv * w; i += blockDim.x) {
        const int g = i / w, e = i % w;
        T* dst = kv_pool + (((size_t)page * nkv + g) * page_size + off) * w;
        if (e >= dk) {
            // a value: copied as it is (the raw key projection, or the projection's own value)
            dst[e] = values_are_keys ? kr[g * dk + e - dk] : vr[g * dv + e - dk];
            continue;
        }
        const int ki = g * dk + e;
        const float inv = norm == 2 ? k_inv : norm == 1 ? head_inv[nh + g] : 1.f;
        float v = to_f32(kr[ki]) * inv;
        if (norm) v *= k_gain[norm == 2 ? ki : e];
        if (e < rot) {
            const int f = e < half ? e : e - half;
            const int j = e < half ? ki + half : ki - half;
            float s, c;
            sincosf(p * inv_freq[f], &s, &c);
            float other = to_f32(kr[j]) * inv;
            if (norm) other *= k_gain[norm == 2 ? j : (e < half ? e + half : e - half)];
            v = e < half ? v * c - other * s : v * c + other * s;
        }
        dst[e] = from_f32<T>(v);
    }
}

// proj: [tokens, row_stride] with q at 0, k at k_off, v at v_off (ignored when values_are_keys, which needs dv == dk).
// q_gain / k_gain: float, dk entries (norm 1) or nh * dk and nkv * dk (norm 2); inv_freq: rot / 2 floats.
PLLM_EXPORT int pllm_normed_qk_kv_write(int dtype, const void* proj, int row_stride, int k_off, int v_off, void* q_out,
                                        const float* q_gain, const float* k_gain, int norm, float eps, float temp_coef,
                                        int temp_every, const float* inv_freq, int rot, const int* positions, const int* slots,
                                        void* kv_pool, int n_tokens, int nh, int nkv, int dk, int dv, int values_are_keys,
                                        int page_size, long long pool_rows, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || rot < 0 || rot > dk || rot % 2) return PLLM_ERR_SIZE;
    if (norm < 0 || norm > 2 || (norm && (!q_gain || !k_gain)) || (rot && !inv_freq) || temp_every < 0) return PLLM_ERR_SIZE;
    if (values_are_keys && dv != dk) return PLLM_ERR_SIZE;
    const size_t smem = (size_t)(nh + nkv) * sizeof(float);
    if (smem > 40 * 1024) return PLLM_ERR_LIMIT;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(normed_qk_kv_write_kernel<T>, dim3(n_tokens), dim3(256), smem, stream, (const T*)proj, row_stride, k_off, v_off,
                       (T*)q_out, q_gain, k_gain, norm, eps, temp_coef, temp_every, inv_freq, rot, positions, slots, (T*)kv_pool, nh,
                       nkv, dk, dv, values_are_keys, page_size, pool_rows, status);
    });
    return launch_status();
}

template <typename T>
__global__ void gate_mul_kernel(T* y, const T* g, int g_stride, int width, long long total, int kind, int per) {
    pdl_launch_dependents();
    pdl_wait(KID_NORMED_QK);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / width;
        const int c = (int)(i % width);
        const float z = to_f32(g[r * g_stride + c / per]);
        const float s = nq_sigmoid(z);
        y[i] = from_f32<T>(to_f32(y[i]) * (kind == 1 ? z * s : s));
    }
}

PLLM_EXPORT int pllm_gate_mul(int dtype, void* y, const void* g, int g_stride, int n_rows, int width, int kind, int per,
                              cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0 || kind < 0 || kind > 1 || per < 1 || width % per) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const long long total = (long long)n_rows * width;
        const int blocks = (int)min((long long)sm_count() * 8, (total + 255) / 256);
        launch_chained(gate_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)y, (const T*)g, g_stride, width, total, kind, per);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(normed_qk)
