// Differential attention, and latent attention with a rotated key part: what lies between their projections and the
// attention kernels, and behind those.
//
//   conv_rope_kv_write   A token's projection row holds [q | k | v] channels.  Each channel (plus its bias) passes a short causal
//                        convolution over the request's tokens, y_t = sum_j w[c, j] x_(t - taps + 1 + j), zeros before the
//                        request's first token; inputs of earlier steps come from the request's state slot
//                        ([taps - 1][channels], oldest first).  Then the first `rot` entries of every q and k head are turned
//                        (entry i with entry i + rot / 2, angle = position * inv_freq[i]); q goes to its own tensor, k | v to
//                        the token's row of the joined pool.  With `maps` > 1 each kv head has that many keys a token (maps of
//                        an attention that takes several softmaxes over the same values): the pool then has kv_heads * maps
//                        rows a token, each a key of its own followed by the kv head's value.
//   conv_state_update    moves the last taps - 1 inputs (projection + bias) of each request into its slot, after the step's
//                        convolutions have read the old ones.
//   diff_combine         o = a_1 - lambda a_2 a head, over its root mean square, times a constant, times sigmoid(gate a head).
//                        The attention's heads arrive ordered [kv head][map][head of the group].
//   latent_rope_write    a token's down-projection [latent | rotated key part]: the latent over its root mean square times a
//                        gain, the key part turned pairwise (entry 2i with 2i + 1), both side by side in the token's cache row;
//                        and the rotated part of every query head turned likewise into the last entries of the query rows that
//                        the attention over cache rows reads.
// Everything is float from the projection's values to the one rounding on the way out.
#include "common.cuh"

enum : int { KID_DIFF = 110 };

#define DA_MAX_TAPS 16

struct DASegment { int first, count, before, slot; };

__device__ __forceinline__ float da_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// grid (segments, chunks of `tok` tokens); conv_w float [channels, taps]; bias float [channels] or null.  A CTA stages the
// inputs (+ bias) of its tokens and of the taps - 1 before them in shared memory, [tok + taps - 1][channels] floats, so that an
// input is fetched once for all the taps that meet it; a thread then keeps one channel's taps (and those of the channel it is
// rotated with) in registers and goes through the chunk's tokens.
template <typename T, int MAXT>       // MAXT >= taps: how many taps a thread keeps in registers
__global__ void __launch_bounds__(512) conv_rope_kv_write_kernel(
    const T* proj, int row_stride, const float* __restrict__ bias, const float* __restrict__ conv_w, int taps,
    const DASegment* __restrict__ segs, const float* state, long long state_stride,
    const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions, const int* __restrict__ slots,
    T* __restrict__ q_out, T* kv_pool, int q_heads, int k_heads, int maps, int dk, int dv, int page_size, long long pool_rows,
    int tok, int* status) {
    extern __shared__ __align__(16) float da_tile[];      // [tok + taps - 1][channels], then [tok][rot / 2] cosines and as many sines
    __shared__ long long base_s[32];                      // where a token's rows begin in the pool (kv head 0), or -1
    pdl_launch_dependents();
    pdl_wait(KID_DIFF);
    const DASegment s = segs[blockIdx.x];
    const int t0 = blockIdx.y * tok;
    if (t0 >= s.count) return;
    const int nt = min(tok, s.count - t0);
    const int cq = q_heads * dk, ck = k_heads * dk, cv = (k_heads / maps) * dv;
    const int channels = cq + ck + cv;
    const int row_w = dk + dv;
    const float* st = state + (size_t)s.slot * state_stride;
    if (threadIdx.x < nt) {
        const int token = s.first + t0 + threadIdx.x;
        const int slot = (kv_pool && slots) ? slots[token] : -1;
        if (slot >= pool_rows) atomicOr(status, 2);
        base_s[threadIdx.x] = (slot >= 0 && slot < pool_rows)
            ? ((long long)(slot / page_size) * k_heads * page_size + slot % page_size) * row_w : -1;
    }
    const int rows = nt + taps - 1;
    const int half = rot / 2;
    // a token's angles are the same for every head: formed once a token and pair
    float* cos_s = da_tile + (size_t)(tok + taps - 1) * channels;
    float* sin_s = cos_s + tok * half;
    for (int idx = threadIdx.x; idx < nt * half; idx += blockDim.x) {
        float sn, cs;
        sincosf((float)positions[s.first + t0 + idx / half] * inv_freq[idx % half], &sn, &cs);
        cos_s[idx] = cs; sin_s[idx] = sn;
    }
    constexpr int N = Vec16<T>::N;
    if (channels % N == 0 && row_stride % N == 0 && ((uintptr_t)proj & 15) == 0) {
        const int vec_per_row = channels / N;
        for (int idx = threadIdx.x; idx < rows * vec_per_row; idx += blockDim.x) {
            const int rr = idx / vec_per_row, c = (idx % vec_per_row) * N;
            const int r = t0 - (taps - 1) + rr;        // relative to the segment's first token
            float f[N];
            if (r >= 0) {
                Vec16<T> v; v.load(proj + (size_t)(s.first + r) * row_stride + c); v.unpack(f);
                if (bias) {
#pragma unroll
                    for (int k = 0; k < N; k += 4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bias + c + k);
                        f[k] += b4.x; f[k + 1] += b4.y; f[k + 2] += b4.z; f[k + 3] += b4.w;
                    }
                }
            } else if (s.before > 0) {
#pragma unroll
                for (int k = 0; k < N; k += 4) {
                    const float4 o4 = *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 + r) * channels + c + k);
                    f[k] = o4.x; f[k + 1] = o4.y; f[k + 2] = o4.z; f[k + 3] = o4.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < N; k++) f[k] = 0.f;
            }
#pragma unroll
            for (int k = 0; k < N; k += 4)
                *reinterpret_cast<float4*>(da_tile + (size_t)rr * channels + c + k) = make_float4(f[k], f[k + 1], f[k + 2], f[k + 3]);
        }
    } else {
        for (int idx = threadIdx.x; idx < rows * channels; idx += blockDim.x) {
            const int rr = idx / channels, c = idx % channels;
            const int r = t0 - (taps - 1) + rr;
            da_tile[idx] = r >= 0 ? to_f32(proj[(size_t)(s.first + r) * row_stride + c]) + (bias ? bias[c] : 0.f)
                                  : (s.before > 0 ? st[(size_t)(taps - 1 + r) * channels + c] : 0.f);
        }
    }
    __syncthreads();
    const long long head_stride = (long long)page_size * row_w;      // from a kv head's rows of a page to the next one's
    for (int i = threadIdx.x; i < channels; i += blockDim.x) {
        // what does not depend on the token: the channel's place in its head, the channel it is turned with, its taps, and
        // where it goes in a token's rows
        const bool is_q = i < cq, is_v = i >= cq + ck;
        const int within = is_v ? i - cq - ck : (is_q ? i : i - cq);
        const int head = within / (is_v ? dv : dk), e = within - head * (is_v ? dv : dk);
        const bool turned = !is_v && e < rot;
        const int eh = turned ? (e < half ? e : e - half) : 0;
        const int partner = turned ? (e < half ? i + half : i - half) : i;
        const float sign = e < half ? -1.f : 1.f;
        const long long off = is_v ? (long long)head * maps * head_stride + dk + e : (long long)head * head_stride + e;
        float wi[MAXT], wp[MAXT];
#pragma unroll
        for (int j = 0; j < MAXT; j++) {
            wi[j] = j < taps ? conv_w[(size_t)i * taps + j] : 0.f;
            wp[j] = (turned && j < taps) ? conv_w[(size_t)partner * taps + j] : 0.f;
        }
        const float* mine = da_tile + i;
        const float* other = da_tile + partner;
        T* qdst = q_out + (size_t)(s.first + t0) * cq + i;
        for (int t = 0; t < nt; t++) {
            float y = 0.f, yp = 0.f;
#pragma unroll
            for (int j = 0; j < MAXT; j++) {        // (taps beyond the convolution's have weight zero and meet the tile's own rows)
                if (j < taps) {
                    y = fmaf(wi[j], mine[(size_t)(t + j) * channels], y);
                    yp = fmaf(wp[j], other[(size_t)(t + j) * channels], yp);
                }
            }
            if (turned) y = y * cos_s[t * half + eh] + sign * yp * sin_s[t * half + eh];
            const T out = from_f32<T>(y);
            if (is_q) qdst[(size_t)t * cq] = out;
            else {
                const long long base = base_s[t];
                if (base >= 0) {
                    if (!is_v) kv_pool[base + off] = out;
                    else
                        for (int z = 0; z < maps; z++) kv_pool[base + off + z * head_stride] = out;      // behind every map's key
                }
            }
        }
    }
}

// grid (segments, channel blocks of 256); a thread a channel, oldest row first: a row is read before it is overwritten.
template <typename T>
__global__ void __launch_bounds__(256) conv_state_update_kernel(const T* proj, int row_stride, const float* __restrict__ bias, int taps,
                                                                const DASegment* __restrict__ segs, float* state,
                                                                long long state_stride, int channels) {
    pdl_launch_dependents();
    pdl_wait(KID_DIFF);
    const DASegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= channels) return;
    float* st = state + (size_t)s.slot * state_stride;
    const float b = bias ? bias[c] : 0.f;
    for (int r = 0; r < taps - 1; r++) {
        const int rel = s.count - (taps - 1) + r;
        float x;
        if (rel >= 0) x = to_f32(proj[(size_t)(s.first + rel) * row_stride + c]) + b;
        else x = s.before > 0 ? st[(size_t)(s.count + r) * channels + c] : 0.f;
        st[(size_t)r * channels + c] = x;
    }
}

PLLM_EXPORT int pllm_conv_rope_kv_write(int dtype, const void* proj, int row_stride, const float* bias, const float* conv_w, int taps,
                                        const int* segs, int n_segs, int max_segment_tokens, float* state, long long state_stride,
                                        const float* inv_freq, int rot, const int* positions, const int* slots, void* q_out,
                                        void* kv_pool, int q_heads, int k_heads, int maps, int dk, int dv, int page_size,
                                        long long pool_rows, int* status, cudaStream_t stream) {
    if (n_segs <= 0 || max_segment_tokens <= 0) return PLLM_OK;
    if (taps < 1 || taps > DA_MAX_TAPS || maps < 1 || k_heads % maps || q_heads <= 0 || dk <= 0 || dv <= 0 || page_size <= 0)
        return PLLM_ERR_SIZE;
    if (rot < 0 || rot % 2 || rot > dk || (rot > 0 && !inv_freq)) return PLLM_ERR_SIZE;
    const int channels = (q_heads + k_heads) * dk + (k_heads / maps) * dv;
    // tokens a CTA: what some 100 KB of shared memory hold beside the taps - 1 rows before them (two CTAs of sixteen warps an
    // SM), 16 at most: what a thread works out for its channel is then shared by several tokens
    const size_t row_bytes = (size_t)channels * sizeof(float);
    if (row_bytes * taps + (size_t)rot * sizeof(float) > 200 * 1024) return PLLM_ERR_LIMIT;
    const int fit = (int)((size_t)(100 * 1024) / row_bytes);      // rows of the tile
    int tok = max(1, min(16, fit - (taps - 1)));
    tok = min(tok, max_segment_tokens);
    const size_t smem = row_bytes * (tok + taps - 1) + (size_t)tok * rot * sizeof(float);
    const int chunks = (max_segment_tokens + tok - 1) / tok;
    if (chunks > 65535) return PLLM_ERR_LIMIT;
#define DA_LAUNCH(MAXT)                                                                                                          \
    do {                                                                                                                         \
        cudaFuncSetAttribute(conv_rope_kv_write_kernel<T, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        launch_chained(conv_rope_kv_write_kernel<T, MAXT>, dim3(n_segs, chunks), dim3(512), smem, stream, (const T*)proj,        \
                       row_stride, bias, conv_w, taps, (const DASegment*)segs, (const float*)state, state_stride, inv_freq, rot, \
                       positions, slots, (T*)q_out, (T*)kv_pool, q_heads, k_heads, maps, dk, dv, page_size, pool_rows, tok,      \
                       status);                                                                                                  \
    } while (0)
    PLLM_DISPATCH_DTYPE(dtype, {
        if (taps <= 4) DA_LAUNCH(4);
        else DA_LAUNCH(DA_MAX_TAPS);
        if (taps > 1)
            launch_chained(conv_state_update_kernel<T>, dim3(n_segs, (channels + 255) / 256), dim3(256), 0, stream, (const T*)proj,
                           row_stride, bias, taps, (const DASegment*)segs, state, state_stride, channels);
    });
#undef DA_LAUNCH
    return launch_status();
}

// a [tokens, kv_heads * 2 * group, dv] (heads ordered [kv head][map][head of the group]); gate [tokens, heads] logits with a row
// stride; y [tokens, heads, dv].  A warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(256) diff_combine_kernel(const T* a, const T* gate, int gate_stride, T* __restrict__ y, long long rows,
                                                           int heads, int group, int dv, float lambda, float post, float eps) {
    pdl_launch_dependents();
    pdl_wait(KID_DIFF);
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const long long t = row / heads;
    const int h = (int)(row % heads), g = h / group, hh = h % group;
    const T* a1 = a + ((size_t)t * 2 * heads + (size_t)(g * 2) * group + hh) * dv;
    const T* a2 = a1 + (size_t)group * dv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) { const float o = to_f32(a1[e]) - lambda * to_f32(a2[e]); ss = fmaf(o, o, ss); }
    ss = warp_sum(ss);
    const float f = post * da_sigmoid(to_f32(gate[(size_t)t * gate_stride + h])) / sqrtf(ss / (float)dv + eps);
    T* out = y + ((size_t)t * heads + h) * dv;
    for (int e = lane; e < dv; e += 32) out[e] = from_f32<T>((to_f32(a1[e]) - lambda * to_f32(a2[e])) * f);
}

PLLM_EXPORT int pllm_diff_combine(int dtype, const void* a, const void* gate, int gate_stride, void* y, int n_tokens, int heads, int group,
                                  int dv, float lambda, float post, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (heads <= 0 || group <= 0 || heads % group || dv <= 0) return PLLM_ERR_SIZE;
    const long long rows = (long long)n_tokens * heads;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(diff_combine_kernel<T>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, stream, (const T*)a, (const T*)gate,
                       gate_stride, (T*)y, rows, heads, group, dv, lambda, post, eps);
    });
    return launch_status();
}

// One CTA a token.  down [tokens, down_stride]: latent (kv_rank) then the key part (rot_dim), or null for a layer that makes
// no rows of its own; row_out [tokens, kv_rank + rot_dim] or null: the rows also go there, for later layers of the step that
// keep copies of them; carried [tokens, kv_rank + rot_dim] or null (with down null): such rows, stored as they are.  q [tokens, q_stride]: a head's entries are [dim | rot_dim]; q_rows [tokens, heads, kv_rank + rot_dim]:
// only the last rot_dim of a head are written here.  The cache row is [kv_rank | rot_dim].
template <typename T>
__global__ void __launch_bounds__(128) latent_rope_write_kernel(const T* down, int down_stride, const float* __restrict__ gain, float eps,
                                                                const T* q, int q_stride, T* __restrict__ q_rows, T* pool,
                                                                T* __restrict__ row_out, const T* __restrict__ carried,
                                                                const int* __restrict__ slots, const int* __restrict__ positions,
                                                                const float* __restrict__ inv_freq, int heads, int dim, int rot_dim,
                                                                int rot, int kv_rank, long long pool_rows, int* status) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait(KID_DIFF);
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    const int width = kv_rank + rot_dim;
    for (int i = threadIdx.x; i < heads * rot_dim; i += blockDim.x) {
        const int h = i / rot_dim, e = i % rot_dim;
        const T* src = q + (size_t)t * q_stride + (size_t)h * (dim + rot_dim) + dim;
        float y = to_f32(src[e]);
        if (e < rot) {
            float sn, cs;
            sincosf(pos * inv_freq[e >> 1], &sn, &cs);
            y = (e & 1) ? y * cs + to_f32(src[e - 1]) * sn : y * cs - to_f32(src[e + 1]) * sn;
        }
        q_rows[((size_t)t * heads + h) * width + kv_rank + e] = from_f32<T>(y);
    }
    const int slot = (pool && slots) ? slots[t] : -1;
    if (!down) {
        if (!carried) return;
        if (slot >= pool_rows && threadIdx.x == 0) atomicOr(status, 2);
        if (slot < 0 || slot >= pool_rows) return;
        for (int c = threadIdx.x; c < width; c += blockDim.x) pool[(size_t)slot * width + c] = carried[(size_t)t * width + c];
        return;
    }
    const T* row = down + (size_t)t * down_stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) { const float v = to_f32(row[c]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    if (slot >= pool_rows && threadIdx.x == 0) atomicOr(status, 2);
    const bool writes = slot >= 0 && slot < pool_rows;
    if (!writes && !row_out) return;
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    T* dst = writes ? pool + (size_t)slot * width : nullptr;
    T* dst2 = row_out ? row_out + (size_t)t * width : nullptr;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const T y = from_f32<T>(to_f32(row[c]) * inv * gain[c]);
        if (dst) dst[c] = y;
        if (dst2) dst2[c] = y;
    }
    for (int e = threadIdx.x; e < rot_dim; e += blockDim.x) {
        float y = to_f32(row[kv_rank + e]);
        if (e < rot) {
            float sn, cs;
            sincosf(pos * inv_freq[e >> 1], &sn, &cs);
            y = (e & 1) ? y * cs + to_f32(row[kv_rank + e - 1]) * sn : y * cs - to_f32(row[kv_rank + e + 1]) * sn;
        }
        if (dst) dst[kv_rank + e] = from_f32<T>(y);
        if (dst2) dst2[kv_rank + e] = from_f32<T>(y);
    }
}

PLLM_EXPORT int pllm_latent_rope_write(int dtype, const void* down, int down_stride, const float* gain, float eps, const void* q,
                                       int q_stride, void* q_rows, void* pool, void* row_out, const void* carried, const int* slots,
                                       const int* positions,
                                       const float* inv_freq, int n_tokens, int heads, int dim, int rot_dim, int rot, int kv_rank,
                                       long long pool_rows, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (heads <= 0 || dim < 0 || rot_dim < 0 || kv_rank <= 0 || rot < 0 || rot % 2 || rot > rot_dim || (rot > 0 && !inv_freq))
        return PLLM_ERR_SIZE;
    if (down && !gain) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(latent_rope_write_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, (const T*)down, down_stride, gain, eps,
                       (const T*)q, q_stride, (T*)q_rows, (T*)pool, (T*)row_out, (const T*)carried, slots, positions, inv_freq, heads,
                       dim, rot_dim, rot, kv_rank, pool_rows, status);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(diff_attention)
