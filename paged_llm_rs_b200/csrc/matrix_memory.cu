// Recurrent mixers whose state is one matrix a head, S (d x e: key entries by value entries), carried from token to token
// in float for every request (a state slot), between their input and output projections.
//
//   matrix LSTM   gates a token and head: i = cap tanh((i_raw + b_i) / cap), f = logsigmoid(cap tanh((f_raw + b_f) / cap));
//                 with a running maximum m (zero at the start):
//                     m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' likewise with k alone
//                     o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
//                 slot: [heads * d * e | heads * d (n) | heads (m)]
//   gated delta   q, k, v pass a short causal convolution a channel (no bias) and silu; q and k become unit vectors a head
//   rule          (x / sqrt(sum x^2 + 1e-6)), q times d^(-1/2); beta = sigmoid(b_raw), g = exp(-exp(A_log) softplus(a_raw + dt_bias))
//                     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                 slot: [heads * d * e | (taps - 1) * channels: the convolution's last inputs, oldest first]
//   head_norm_gate   each head's o over its root mean square, times a gain (one a head entry, or shared by the heads), times
//                    sigmoid or silu of a gate: the output projection's input
//
// A step is a list of segments {first token, tokens, tokens before, state slot} on the device; grids are sized by the list's
// capacity and a segment of no tokens does nothing, so a captured step replays for any step that fits.
// A thread holds rows part, part + PARTS, ... of ONE column of S; the PARTS threads of a column are neighbours in a warp and
// meet by shuffles in a fixed order, columns never meet: what a token's output is does not depend on how the columns are
// shared out among CTAs, nor on where a prompt was cut.
#include "common.cuh"

enum : int { KID_MATRIX_MEMORY = 100 };

#define MM_CHUNK 32            // tokens fetched at a time (fewer where keys are so long that shared memory would not hold them)
#define MM_CONV_TOKENS 64      // tokens a CTA of the convolution
#define MM_MAX_TAPS 16

struct MMSegment { int first, count, before, slot; };

__device__ __forceinline__ float mm_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float mm_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float mm_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float mm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float mm_parts_sum(float v, int parts) {
    for (int o = parts >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// grid (segments, channel blocks of 128, token chunks); u: [tokens, u_width] with the channels at u_off; conv_w [channels, taps],
// the last tap meets the current token.
template <typename T>
__global__ void __launch_bounds__(128) mm_conv_silu_kernel(const T* u, int u_width, int u_off, const T* __restrict__ conv_w,
                                                           const MMSegment* __restrict__ segs, const float* state, long long state_stride,
                                                           long long conv_off, float* __restrict__ c_out, int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    const int t0 = blockIdx.z * MM_CONV_TOKENS;
    if (t0 >= s.count) return;
    const int ch = blockIdx.y * 128 + threadIdx.x;
    if (ch >= channels) return;
    float wt[MM_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MM_MAX_TAPS; j++) wt[j] = j < taps ? to_f32(conv_w[(size_t)ch * taps + j]) : 0.f;
    const float* st = state + (size_t)s.slot * state_stride + conv_off;       // [taps - 1][channels], oldest first
    const int t1 = min(s.count, t0 + MM_CONV_TOKENS);
    for (int t = t0; t < t1; t++) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < MM_MAX_TAPS; j++) {
            if (j >= taps) break;
            const int r = t - (taps - 1) + j;              // relative to the segment's first token
            float v;
            if (r >= 0) v = to_f32(u[(size_t)(s.first + r) * u_width + u_off + ch]);
            else v = s.before > 0 ? st[(size_t)(taps - 1 + r) * channels + ch] : 0.f;
            acc = fmaf(wt[j], v, acc);
        }
        c_out[(size_t)(s.first + t) * channels + ch] = mm_silu(acc);
    }
}

// grid (segments, heads, slices of e); thread (col, part) = (tid / PARTS, tid % PARTS) holds rows part + k PARTS of column
// p0 + col.  c: [tokens, channels] float, q at 0 (G d), k at G d, v at 2 G d (H e).  ba: [tokens, 2 H] float, b_raw | a_raw.
// u (the projection, for the convolution's state): [tokens, u_width] with the channels at conv_in_off.
template <typename T, int NPT>
__global__ void __launch_bounds__(256) delta_scan_kernel(const float* c, int channels, const float* ba, const T* u, int u_width, int conv_in_off,
                                                         const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                                         const MMSegment* __restrict__ segs, float* state, long long state_stride,
                                                         long long conv_off, float* __restrict__ y, int H, int G, int d, int E, int Ps,
                                                         int parts, int taps, int ck) {
    extern __shared__ float mm_smem[];
    const int NP = NPT * parts;
    float* q_s = mm_smem;                        // [ck][NP]
    float* k_s = q_s + ck * NP;            // [ck][NP]
    float* v_s = k_s + ck * NP;            // [ck][Ps]
    float* g_s = v_s + ck * Ps;            // [ck] decay, then [ck] beta
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, kh = h / (H / G), p0 = blockIdx.z * Ps;
    const int col = threadIdx.x / parts, part = threadIdx.x % parts;
    const int e = p0 + col;
    const bool live = col < Ps && e < E;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* S = state + (size_t)s.slot * state_stride + (size_t)h * d * E;
    float st[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part + k * parts;
        st[k] = (live && n < d && s.before > 0) ? S[(size_t)n * E + e] : 0.f;
    }
    const float A = -expf(a_log[h]), bias = dt_bias[h];
    const float q_scale = rsqrtf((float)d);
    for (int i = threadIdx.x; i < 2 * ck * NP; i += blockDim.x) q_s[i] = 0.f;      // (the padding rows stay zero)
    for (int t0 = 0; t0 < s.count; t0 += ck) {
        const int nt = min(ck, s.count - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * d; i += blockDim.x) {
            const float* row = c + (size_t)(s.first + t0 + i / d) * channels + kh * d + i % d;
            q_s[(i / d) * NP + i % d] = row[0];
            k_s[(i / d) * NP + i % d] = row[(size_t)G * d];
        }
        for (int i = threadIdx.x; i < nt * Ps; i += blockDim.x) {
            const int ee = p0 + i % Ps;
            v_s[i] = ee < E ? c[(size_t)(s.first + t0 + i / Ps) * channels + 2 * G * d + h * E + ee] : 0.f;
        }
        if (threadIdx.x < nt) {
            const float* r = ba + (size_t)(s.first + t0 + threadIdx.x) * 2 * H;
            g_s[threadIdx.x] = expf(A * mm_softplus(r[H + h] + bias));
            g_s[ck + threadIdx.x] = mm_sigmoid(r[h]);
        }
        __syncthreads();
        // unit vectors: a warp a token
        for (int t = warp; t < nt; t += warps) {
            float sq = 0.f, sk = 0.f;
            for (int n = lane; n < d; n += 32) { const float a = q_s[t * NP + n], b = k_s[t * NP + n]; sq += a * a; sk += b * b; }
            sq = warp_sum(sq); sk = warp_sum(sk);
            const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
            for (int n = lane; n < d; n += 32) { q_s[t * NP + n] *= iq; k_s[t * NP + n] *= ik; }
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float g = g_s[t], beta = g_s[ck + t];
            const float v = col < Ps ? v_s[t * Ps + col] : 0.f;
            const float* kt = k_s + t * NP + part;
            const float* qt = q_s + t * NP + part;
            float kk[NPT];
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                kk[k] = kt[k * parts];
                st[k] *= g;
                if (k & 1) a1 = fmaf(st[k], kk[k], a1); else a0 = fmaf(st[k], kk[k], a0);
            }
            const float uu = beta * (v - mm_parts_sum(a0 + a1, parts));
            a0 = 0.f; a1 = 0.f;
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                st[k] = fmaf(kk[k], uu, st[k]);
                const float qq = qt[k * parts];
                if (k & 1) a1 = fmaf(st[k], qq, a1); else a0 = fmaf(st[k], qq, a0);
            }
            const float o = mm_parts_sum(a0 + a1, parts);
            if (live && part == 0) y[(size_t)(s.first + t0 + t) * H * E + h * E + e] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int k = 0; k < NPT; k++) {
            const int n = part + k * parts;
            if (n < d) S[(size_t)n * E + e] = st[k];
        }
    }
    // The convolution's state: the last taps - 1 inputs of this CTA's value channels, and of its kv head's q and k channels by
    // the kv head's first head and first slice.  The convolution kernel has finished; nobody else touches these channels.
    float* cs = state + (size_t)s.slot * state_stride + conv_off;
    const int hpg = H / G;
    const int extra = (h % hpg == 0 && blockIdx.z == 0) ? 2 * d : 0;
    const int nv = min(Ps, E - p0);
    for (int i = threadIdx.x; i < nv + extra; i += blockDim.x) {
        int ch;
        if (i < nv) ch = 2 * G * d + h * E + p0 + i;
        else if (i < nv + d) ch = kh * d + (i - nv);
        else ch = G * d + kh * d + (i - nv - d);
        float keep[MM_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < MM_MAX_TAPS; k++) {
            if (k >= taps - 1) break;
            const int r = s.count - (taps - 1) + k;
            if (r >= 0) keep[k] = to_f32(u[(size_t)(s.first + r) * u_width + conv_in_off + ch]);
            else keep[k] = s.before > 0 ? cs[(size_t)(taps - 1 + r) * channels + ch] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < MM_MAX_TAPS; k++) {
            if (k >= taps - 1) break;
            cs[(size_t)k * channels + ch] = keep[k];
        }
    }
}

// grid and threads as above.  u: [tokens, u_width] of the compute dtype, q at 0 (H d), k at H d, v at 2 H d (H e).
// gates: [tokens, 2 H] float, i_raw | f_raw.
template <typename T, int NPT>
__global__ void __launch_bounds__(256) mlstm_scan_kernel(const T* u, int u_width, const float* gates, const float* __restrict__ i_bias,
                                                         const float* __restrict__ f_bias, float cap, const MMSegment* __restrict__ segs,
                                                         float* state, long long state_stride, float* __restrict__ nm_buf,
                                                         float* __restrict__ y, int H, int d, int E, int Ps, int parts, int ck) {
    extern __shared__ float mm_smem[];
    const int NP = NPT * parts;
    float* q_s = mm_smem;                        // [ck][NP]
    float* k_s = q_s + ck * NP;            // [ck][NP]
    float* v_s = k_s + ck * NP;            // [ck][Ps]
    float* a_s = v_s + ck * Ps;            // [ck] exp(f + m - m'), then [ck] exp(i - m'), then [ck] exp(-m')
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, p0 = blockIdx.z * Ps;
    const int col = threadIdx.x / parts, part = threadIdx.x % parts;
    const int e = p0 + col;
    const bool live = col < Ps && e < E;
    float* slot = state + (size_t)s.slot * state_stride;
    float* S = slot + (size_t)h * d * E;
    float* n_st = slot + (size_t)H * d * E + (size_t)h * d;
    float* m_st = slot + (size_t)H * d * E + (size_t)H * d + h;
    float st[NPT], nn[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part + k * parts;
        const bool have = n < d && s.before > 0;
        st[k] = (live && have) ? S[(size_t)n * E + e] : 0.f;
        nn[k] = have ? n_st[n] : 0.f;
    }
    float m = s.before > 0 ? *m_st : 0.f;        // (used by thread 0 only)
    const float bi = i_bias[h], bf = f_bias[h];
    const float q_scale = rsqrtf((float)d);
    for (int i = threadIdx.x; i < 2 * ck * NP; i += blockDim.x) q_s[i] = 0.f;      // (the padding rows stay zero)
    for (int t0 = 0; t0 < s.count; t0 += ck) {
        const int nt = min(ck, s.count - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * d; i += blockDim.x) {
            const T* row = u + (size_t)(s.first + t0 + i / d) * u_width + h * d + i % d;
            q_s[(i / d) * NP + i % d] = to_f32(row[0]) * q_scale;
            k_s[(i / d) * NP + i % d] = to_f32(row[(size_t)H * d]);
        }
        for (int i = threadIdx.x; i < nt * Ps; i += blockDim.x) {
            const int ee = p0 + i % Ps;
            v_s[i] = ee < E ? to_f32(u[(size_t)(s.first + t0 + i / Ps) * u_width + 2 * H * d + h * E + ee]) : 0.f;
        }
        if (threadIdx.x < nt) {
            const float* r = gates + (size_t)(s.first + t0 + threadIdx.x) * 2 * H;
            a_s[threadIdx.x] = mm_logsigmoid(cap * tanhf((r[H + h] + bf) / cap));
            a_s[ck + threadIdx.x] = cap * tanhf((r[h] + bi) / cap);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // the running maximum goes from token to token: one thread, over values that are already in shared memory
            for (int t = 0; t < nt; t++) {
                const float fg = a_s[t], ig = a_s[ck + t];
                const float m_new = fmaxf(fg + m, ig);
                a_s[t] = expf(fg + m - m_new);
                a_s[ck + t] = expf(ig - m_new);
                a_s[2 * ck + t] = expf(-m_new);
                m = m_new;
            }
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float a = a_s[t], b = a_s[ck + t], em = a_s[2 * ck + t];
            const float bv = b * (col < Ps ? v_s[t * Ps + col] : 0.f);
            const float* kt = k_s + t * NP + part;
            const float* qt = q_s + t * NP + part;
            float num0 = 0.f, num1 = 0.f, den0 = 0.f, den1 = 0.f;
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                const float kk = kt[k * parts], qq = qt[k * parts];
                st[k] = fmaf(a, st[k], kk * bv);
                nn[k] = fmaf(a, nn[k], kk * b);
                if (k & 1) { num1 = fmaf(st[k], qq, num1); den1 = fmaf(nn[k], qq, den1); }
                else { num0 = fmaf(st[k], qq, num0); den0 = fmaf(nn[k], qq, den0); }
            }
            const float num = mm_parts_sum(num0 + num1, parts), den = mm_parts_sum(den0 + den1, parts);
            if (live && part == 0) y[(size_t)(s.first + t0 + t) * H * E + h * E + e] = num / (fmaxf(fabsf(den), em) + 1e-6f);
        }
    }
    // Every slice of a head reads the head's n and m when it starts, and slices start at different times: the new n and m
    // go to a scratch row of the step, and the kernel behind this one moves them into the slot.
    float* nm = nm_buf + ((size_t)blockIdx.x * H + h) * (d + 1);
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part + k * parts;
        if (n < d) {
            if (live) S[(size_t)n * E + e] = st[k];
            if (blockIdx.z == 0 && col == 0) nm[n] = nn[k];
        }
    }
    if (blockIdx.z == 0 && threadIdx.x == 0) nm[d] = m;
}

// grid (segments, heads): a head's new normaliser and running maximum from the step's scratch into the request's slot.
__global__ void __launch_bounds__(128) mlstm_store_nm_kernel(const float* __restrict__ nm_buf, const MMSegment* __restrict__ segs,
                                                             float* state, long long state_stride, int H, int d, int E) {
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y;
    const float* nm = nm_buf + ((size_t)blockIdx.x * H + h) * (d + 1);
    float* slot = state + (size_t)s.slot * state_stride;
    for (int n = threadIdx.x; n < d; n += blockDim.x) slot[(size_t)H * d * E + (size_t)h * d + n] = nm[n];
    if (threadIdx.x == 0) slot[(size_t)H * d * E + (size_t)H * d + h] = nm[d];
}

// A warp a (token, head): o / rms(o) * gain * act(gate).  y float [tokens, H e]; gate: [tokens, g_stride] of the compute dtype;
// gain_per_head: the gain has H e entries, else e entries shared by the heads; kind 0 sigmoid, 1 silu.
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* y, const T* gate, int g_stride, const float* __restrict__ gain,
                                                             T* __restrict__ out, long long n_rows, int H, int E, int gain_per_head,
                                                             int kind, float eps) {
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const int lane = threadIdx.x & 31;
    const long long r = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long t = r / H;
    const int h = (int)(r % H);
    const float* yr = y + r * E;
    const T* gr = gate + t * g_stride + (size_t)h * E;
    float ss = 0.f;
    for (int i = lane; i < E; i += 32) { const float v = yr[i]; ss += v * v; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps);
    for (int i = lane; i < E; i += 32) {
        const float z = to_f32(gr[i]);
        const float sg = mm_sigmoid(z);
        out[r * E + i] = from_f32<T>(yr[i] * inv * gain[gain_per_head ? h * E + i : i] * (kind == 1 ? z * sg : sg));
    }
}

struct MMShape { int parts, npt, Ps, slices, threads, chunk; size_t smem; };

// How a head's state is shared out: PARTS threads a column so that a thread holds at most 16 rows (32 for the longest
// keys), columns a CTA so that a CTA has some 128 threads, fewer where that puts the step on more SMs.
static inline int mm_shape(int n_segs, int H, int d, int E, int extra_floats, MMShape* out) {
    int parts = 1;
    while (parts < 32 && (d + parts - 1) / parts > 16) parts *= 2;
    const int rows = (d + parts - 1) / parts;
    if (rows > 32) return PLLM_ERR_LIMIT;
    const int npt = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    int Ps = 1;
    while (Ps * 2 * parts <= 128 && Ps < E) Ps *= 2;
    while (Ps * parts > 32 && (long long)n_segs * H * ((E + Ps - 1) / Ps) < sm_count()) Ps /= 2;
    out->parts = parts; out->npt = npt; out->Ps = Ps; out->slices = (E + Ps - 1) / Ps;
    out->threads = (Ps * parts + 31) / 32 * 32;
    int chunk = MM_CHUNK;
    auto smem_of = [&](int ck) { return (size_t)ck * (2 * npt * parts + Ps + extra_floats) * sizeof(float); };
    while (chunk > 4 && smem_of(chunk) > 64 * 1024) chunk /= 2;
    out->chunk = chunk;
    out->smem = smem_of(chunk);
    return out->smem > 200 * 1024 ? PLLM_ERR_LIMIT : PLLM_OK;
}

template <typename T>
static void launch_head_norm_gate(const float* y, const void* gate, int g_stride, const float* gain, void* out, int n_tokens, int H, int E,
                                  int gain_per_head, int kind, float eps, cudaStream_t stream) {
    const long long rows = (long long)n_tokens * H;
    launch_chained(head_norm_gate_kernel<T>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, stream, y, (const T*)gate, g_stride, gain,
                   (T*)out, rows, H, E, gain_per_head, kind, eps);
}

#define MM_NPT_DISPATCH(npt, CALL) do { if ((npt) == 4) { constexpr int NPT = 4; CALL; } else if ((npt) == 8) { constexpr int NPT = 8; CALL; } \
    else if ((npt) == 16) { constexpr int NPT = 16; CALL; } else { constexpr int NPT = 32; CALL; } } while (0)

PLLM_EXPORT long long pllm_mlstm_state_floats(int H, int d, int E) { return (long long)H * d * E + (long long)H * d + H; }
PLLM_EXPORT long long pllm_delta_state_floats(int H, int G, int d, int E, int taps) {
    return (long long)H * d * E + (long long)(taps - 1) * (2 * G * d + H * E);
}

// u: [tokens, u_width] of the compute dtype: q (H d) | k (H d) | v (H e) | gate (H e); gates: [tokens, 2 H] float, i_raw | f_raw;
// gain: H e floats; nm_buf: [n_segs, H, d + 1] float scratch; y_buf: [tokens, H e] float scratch; out: [tokens, H e] of the compute dtype.
PLLM_EXPORT int pllm_mlstm_mix(int dtype, const void* u, int u_width, const float* gates, const float* i_bias, const float* f_bias,
                               float cap, const float* gain, const int* segs, int n_segs, float* state, long long state_stride,
                               float* nm_buf, float* y_buf, void* out, int n_tokens, int H, int d, int E, float eps, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return PLLM_OK;
    if (H <= 0 || d <= 0 || E <= 0 || !(cap > 0.f) || u_width < 2 * H * d + 2 * H * E) return PLLM_ERR_SIZE;
    if (state_stride < pllm_mlstm_state_floats(H, d, E)) return PLLM_ERR_SIZE;
    MMShape sh;
    const int rc = mm_shape(n_segs, H, d, E, 3, &sh);
    if (rc != PLLM_OK) return rc;
    PLLM_DISPATCH_DTYPE(dtype, {
        MM_NPT_DISPATCH(sh.npt, {
            if (sh.smem > 48 * 1024)
                cudaFuncSetAttribute(mlstm_scan_kernel<T, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh.smem);
            launch_chained(mlstm_scan_kernel<T, NPT>, dim3(n_segs, H, sh.slices), dim3(sh.threads), sh.smem, stream, (const T*)u, u_width,
                           gates, i_bias, f_bias, cap, (const MMSegment*)segs, state, state_stride, nm_buf, y_buf, H, d, E, sh.Ps, sh.parts,
                           sh.chunk);
        });
        launch_chained(mlstm_store_nm_kernel, dim3(n_segs, H), dim3(128), 0, stream, (const float*)nm_buf, (const MMSegment*)segs, state,
                       state_stride, H, d, E);
        launch_head_norm_gate<T>(y_buf, (const T*)u + 2 * H * d + H * E, u_width, gain, out, n_tokens, H, E, 1, 0, eps, stream);
    });
    return launch_status();
}

// u: [tokens, u_width] of the compute dtype: q (G d) | k (G d) | v (H e) | gate (H e); conv_w: [2 G d + H e, taps] of the same;
// ba: [tokens, 2 H] float, b_raw | a_raw; a_log, dt_bias: H floats; gain: e floats; c_buf [tokens, 2 G d + H e] and
// y_buf [tokens, H e] float scratch; out: [tokens, H e] of the compute dtype.
PLLM_EXPORT int pllm_delta_mix(int dtype, const void* u, int u_width, const void* conv_w, const float* ba, const float* a_log,
                               const float* dt_bias, const float* gain, const int* segs, int n_segs, int max_segment_tokens,
                               float* state, long long state_stride, float* c_buf, float* y_buf, void* out, int n_tokens, int H, int G,
                               int d, int E, int taps, float eps, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return PLLM_OK;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || E <= 0 || taps < 1) return PLLM_ERR_SIZE;
    if (taps > MM_MAX_TAPS) return PLLM_ERR_LIMIT;
    const int channels = 2 * G * d + H * E;
    if (u_width < channels + H * E || state_stride < pllm_delta_state_floats(H, G, d, E, taps)) return PLLM_ERR_SIZE;
    const long long conv_off = (long long)H * d * E;
    MMShape sh;
    const int rc = mm_shape(n_segs, H, d, E, 2, &sh);
    if (rc != PLLM_OK) return rc;
    const int chunks = (max_segment_tokens + MM_CONV_TOKENS - 1) / MM_CONV_TOKENS;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(mm_conv_silu_kernel<T>, dim3(n_segs, (channels + 127) / 128, chunks > 0 ? chunks : 1), dim3(128), 0, stream,
                       (const T*)u, u_width, 0, (const T*)conv_w, (const MMSegment*)segs, (const float*)state, state_stride, conv_off,
                       c_buf, channels, taps);
        MM_NPT_DISPATCH(sh.npt, {
            if (sh.smem > 48 * 1024)
                cudaFuncSetAttribute(delta_scan_kernel<T, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh.smem);
            launch_chained(delta_scan_kernel<T, NPT>, dim3(n_segs, H, sh.slices), dim3(sh.threads), sh.smem, stream, (const float*)c_buf,
                           channels, ba, (const T*)u, u_width, 0, a_log, dt_bias, (const MMSegment*)segs, state, state_stride, conv_off,
                           y_buf, H, G, d, E, sh.Ps, sh.parts, taps, sh.chunk);
        });
        launch_head_norm_gate<T>(y_buf, (const T*)u + channels, u_width, gain, out, n_tokens, H, E, 0, 1, eps, stream);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(matrix_memory)
