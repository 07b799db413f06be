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
// A thread holds some rows of ONE column of S in registers.  Delta rule: rows part, part + PARTS, ...; the PARTS threads of a
// column are neighbours in a warp and meet by shuffles in a fixed order before every write.  Matrix LSTM: rows part NPT ...;
// a column's threads never meet, their shares of a read-out are added in the order of the parts once a chunk.  Columns never
// meet: what a token's output is does not depend on how the columns are shared out among CTAs, and on where a prompt was
// cut only by the rounding of the delta rule's pairs of tokens.  Other threads of the CTA fetch the tokens ahead of the
// recurrence.
#include "common.cuh"

enum : int { KID_MATRIX_MEMORY = 100 };

#define MM_CHUNK 32            // tokens fetched at a time (fewer where keys are so long that shared memory would not hold them)
#define MM_CHUNK_SMALL 8       // ... in a step of decoded tokens
#define MM_CONV_TOKENS 64      // tokens a CTA of the convolution
#define MM_MAX_TAPS 16

struct MMSegment { int first, count, before, slot; };

__device__ __forceinline__ float mm_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float mm_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float mm_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float mm_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float mm_parts_sum(float v, int parts) {
    if (parts > 16) v += __shfl_xor_sync(0xffffffffu, v, 16);
    if (parts > 8) v += __shfl_xor_sync(0xffffffffu, v, 8);
    if (parts > 4) v += __shfl_xor_sync(0xffffffffu, v, 4);
    if (parts > 2) v += __shfl_xor_sync(0xffffffffu, v, 2);
    if (parts > 1) v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}
// two sums at once: the second one's shuffles travel while the first one's are added
__device__ __forceinline__ void mm_parts_sum2(float& a, float& b, int parts) {
    if (parts > 16) { const float x = __shfl_xor_sync(0xffffffffu, a, 16), y = __shfl_xor_sync(0xffffffffu, b, 16); a += x; b += y; }
    if (parts > 8) { const float x = __shfl_xor_sync(0xffffffffu, a, 8), y = __shfl_xor_sync(0xffffffffu, b, 8); a += x; b += y; }
    if (parts > 4) { const float x = __shfl_xor_sync(0xffffffffu, a, 4), y = __shfl_xor_sync(0xffffffffu, b, 4); a += x; b += y; }
    if (parts > 2) { const float x = __shfl_xor_sync(0xffffffffu, a, 2), y = __shfl_xor_sync(0xffffffffu, b, 2); a += x; b += y; }
    if (parts > 1) { const float x = __shfl_xor_sync(0xffffffffu, a, 1), y = __shfl_xor_sync(0xffffffffu, b, 1); a += x; b += y; }
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

// Both recurrences run as two kinds of threads in one CTA.  The first `workers` threads hold the state: thread (col, part) =
// (tid / PARTS, tid % PARTS) has rows part + k PARTS of column p0 + col and goes through a chunk's tokens one after the other.
// The MM_LOADERS threads behind them fetch the NEXT chunk meanwhile (16 bytes a load where the rows allow it), and do what a
// token needs ahead of its step and does not depend on the state: unit vectors, decays, the running maximum.  Two buffers in
// shared memory; one __syncthreads a chunk hands them over.
#define MM_LOADERS 128           // threads that fetch, in a step with a prompt's portion
#define MM_LOADERS_SMALL 32      // ... in a step of decoded tokens

__device__ __forceinline__ void mm_loader_barrier(int loaders) { asm volatile("bar.sync 1, %0;\n" ::"r"(loaders) : "memory"); }

template <typename T> struct MMVec;
template <> struct MMVec<float> { static constexpr int N = 4; };
template <> struct MMVec<bf16> { static constexpr int N = 8; };

// 16 bytes at p (on a 16-byte boundary), times scale, as floats to shared memory (dst on a 16-byte boundary)
__device__ __forceinline__ void mm_fetch16(const float* p, float* dst, float scale) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    *reinterpret_cast<float4*>(dst) = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
}
__device__ __forceinline__ void mm_fetch16(const bf16* p, float* dst, float scale) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(r.x << 16) * scale, __uint_as_float(r.x & 0xffff0000u) * scale,
                                                  __uint_as_float(r.y << 16) * scale, __uint_as_float(r.y & 0xffff0000u) * scale);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(r.z << 16) * scale, __uint_as_float(r.z & 0xffff0000u) * scale,
                                                      __uint_as_float(r.w << 16) * scale, __uint_as_float(r.w & 0xffff0000u) * scale);
}

// grid (segments, heads, slices of e).  c: [tokens, channels] float, q at 0 (G d), k at G d, v at 2 G d (H e).
// ba: [tokens, 2 H] float, b_raw | a_raw.  u (the projection, for the convolution's state): [tokens, u_width] with the
// channels at conv_in_off.
// MINB: CTAs an SM the registers are bounded for (one where the step has no more CTAs than SMs, or a thread holds 32 rows:
// the registers the recurrence likes; else two, for the short CTAs of decoded tokens to overlap)
template <typename T, int NPT, int MINB>
__global__ void __launch_bounds__(256, MINB) delta_scan_kernel(const float* __restrict__ c, int channels, const float* __restrict__ ba, const T* u,
                                                         int u_width, int conv_in_off, const float* __restrict__ a_log,
                                                         const float* __restrict__ dt_bias, const MMSegment* __restrict__ segs, float* state,
                                                         long long state_stride, long long conv_off, float* __restrict__ y, int H, int G,
                                                         int d, int E, int Ps, int parts, int taps, int ck, int workers, int loaders) {
    extern __shared__ __align__(16) float mm_smem[];
    const int NP = NPT * parts;
    // a buffer: q [ck][NP] | k [ck][NP] | v [ck][Ps] | decay [ck] | beta [ck] | k . q [ck] | k . next k [ck] | k . next q [ck]
    const int BUF = ck * (2 * NP + Ps + 5);
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, kh = h / (H / G), p0 = blockIdx.z * Ps;
    const bool loader = (int)threadIdx.x >= workers;
    const int ltid = (int)threadIdx.x - workers;
    const int col = threadIdx.x / parts, part = threadIdx.x % parts;
    const int e = p0 + col;
    const bool live = !loader && col < Ps && e < E;
    float* S = state + (size_t)s.slot * state_stride + (size_t)h * d * E;
    float st[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part + k * parts;
        st[k] = (live && n < d && s.before > 0) ? S[(size_t)n * E + e] : 0.f;
    }
    const float A = -expf(a_log[h]), bias = dt_bias[h];
    const float q_scale = rsqrtf((float)d);
    const bool vec = d % 4 == 0 && channels % 4 == 0 && (reinterpret_cast<uintptr_t>(c) & 15) == 0;
    if (NP > d) {                                   // (the padding rows stay zero)
        for (int b = 0; b < 2; b++)
            for (int i = threadIdx.x; i < 2 * ck * NP; i += blockDim.x) mm_smem[b * BUF + i] = 0.f;
        __syncthreads();
    }
    const int n_chunks = (s.count + ck - 1) / ck;
    for (int cc = -1; cc < n_chunks; cc++) {
        if (loader) {
            if (cc + 1 < n_chunks) {
                const int t0 = (cc + 1) * ck, nt = min(ck, s.count - t0);
                float* q_s = mm_smem + ((cc + 1) & 1) * BUF;
                float* k_s = q_s + ck * NP;
                float* v_s = k_s + ck * NP;
                float* g_s = v_s + ck * Ps;
                // every load of the chunk leaves before the first one is waited for
                float rb = 0.f, ra = 0.f;
                if (ltid < nt) {
                    const float* r = ba + (size_t)(s.first + t0 + ltid) * 2 * H;
                    rb = r[h]; ra = r[H + h];
                }
                float rv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = ltid + j * loaders, ee = p0 + i % Ps;
                    rv[j] = (i < nt * Ps && ee < E) ? c[(size_t)(s.first + t0 + i / Ps) * channels + 2 * G * d + h * E + ee] : 0.f;
                }
                if (vec) {
                    const int dv = d >> 2;
#pragma unroll 8
                    for (int i = ltid; i < nt * dv; i += loaders) {
                        const int t = i / dv, j = (i - t * dv) * 4;
                        const float* row = c + (size_t)(s.first + t0 + t) * channels + kh * d + j;
                        mm_fetch16(row, q_s + t * NP + j, 1.f);
                        mm_fetch16(row + (size_t)G * d, k_s + t * NP + j, 1.f);
                    }
                } else {
                    for (int i = ltid; i < nt * d; i += loaders) {
                        const float* row = c + (size_t)(s.first + t0 + i / d) * channels + kh * d + i % d;
                        q_s[(i / d) * NP + i % d] = row[0];
                        k_s[(i / d) * NP + i % d] = row[(size_t)G * d];
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = ltid + j * loaders;
                    if (i < nt * Ps) v_s[i] = rv[j];
                }
                for (int i = ltid + 4 * loaders; i < nt * Ps; i += loaders) {
                    const int ee = p0 + i % Ps;
                    v_s[i] = ee < E ? c[(size_t)(s.first + t0 + i / Ps) * channels + 2 * G * d + h * E + ee] : 0.f;
                }
                if (ltid < nt) {
                    g_s[ltid] = expf(A * mm_softplus(ra + bias));
                    g_s[ck + ltid] = mm_sigmoid(rb);
                }
                mm_loader_barrier(loaders);
                // unit vectors: a warp a token
                const int lane = ltid & 31;
                for (int t = ltid >> 5; t < nt; t += (loaders >> 5)) {
                    float sq = 0.f, sk = 0.f;
                    for (int n = lane; n < d; n += 32) { const float a = q_s[t * NP + n], b = k_s[t * NP + n]; sq += a * a; sk += b * b; }
                    sq = warp_sum(sq); sk = warp_sum(sk);
                    const float iq = q_scale / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
                    float kq = 0.f;
                    for (int n = lane; n < d; n += 32) {
                        const float a = q_s[t * NP + n] * iq, b = k_s[t * NP + n] * ik;
                        q_s[t * NP + n] = a; k_s[t * NP + n] = b;
                        kq = fmaf(a, b, kq);
                    }
                    kq = warp_sum(kq);
                    if (lane == 0) g_s[2 * ck + t] = kq;
                }
                mm_loader_barrier(loaders);
                // what a pair of tokens taken in one go needs: the first one's key with the second one's key and query
                for (int t = 2 * (ltid >> 5); t + 1 < nt; t += 2 * ((loaders >> 5))) {
                    float kk2 = 0.f, kq2 = 0.f;
                    for (int n = lane; n < d; n += 32) {
                        const float a = k_s[t * NP + n];
                        kk2 = fmaf(a, k_s[(t + 1) * NP + n], kk2); kq2 = fmaf(a, q_s[(t + 1) * NP + n], kq2);
                    }
                    kk2 = warp_sum(kk2); kq2 = warp_sum(kq2);
                    if (lane == 0) { g_s[3 * ck + t] = kk2; g_s[4 * ck + t] = kq2; }
                }
            }
        } else if (cc >= 0) {
            const int t0 = cc * ck, nt = min(ck, s.count - t0);
            const float* q_s = mm_smem + (cc & 1) * BUF;
            const float* k_s = q_s + ck * NP;
            const float* v_s = k_s + ck * NP;
            const float* g_s = v_s + ck * Ps;
            // Two tokens in one go: with S1 = g1 S0 + k1 u1^T, the second token's S1^T k2 = g1 S0^T k2 + u1 (k1 . k2) and
            // S1^T q2 likewise, so all four products are taken with S0 and a column's threads meet once for two tokens.
            int t = 0;
            for (; t + 1 < nt; t += 2) {
                const float g1 = g_s[t], beta1 = g_s[ck + t], kq1 = g_s[2 * ck + t], k1k2 = g_s[3 * ck + t], k1q2 = g_s[4 * ck + t];
                const float g2 = g_s[t + 1], beta2 = g_s[ck + t + 1], kq2 = g_s[2 * ck + t + 1];
                const float v1 = col < Ps ? v_s[t * Ps + col] : 0.f, v2 = col < Ps ? v_s[(t + 1) * Ps + col] : 0.f;
                const float* kt = k_s + t * NP + part;
                const float* qt = q_s + t * NP + part;
                float k1[NPT], k2[NPT];
                float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                for (int k = 0; k < NPT; k++) {
                    k1[k] = kt[k * parts]; k2[k] = kt[NP + k * parts];
                    const float q1 = qt[k * parts], q2 = qt[NP + k * parts];
                    a0 = fmaf(st[k], k1[k], a0); a1 = fmaf(st[k], q1, a1);
                    b0 = fmaf(st[k], k2[k], b0); b1 = fmaf(st[k], q2, b1);
                }
                mm_parts_sum2(a0, a1, parts);
                mm_parts_sum2(b0, b1, parts);
                const float u1 = beta1 * (v1 - g1 * a0);
                const float u2 = beta2 * (v2 - g2 * fmaf(u1, k1k2, g1 * b0));
#pragma unroll
                for (int k = 0; k < NPT; k++) st[k] = fmaf(k2[k], u2, g2 * fmaf(k1[k], u1, g1 * st[k]));
                if (live && part == 0) {
                    float* yo = y + (size_t)(s.first + t0 + t) * H * E + h * E + e;
                    yo[0] = fmaf(u1, kq1, g1 * a1);
                    yo[(size_t)H * E] = fmaf(u2, kq2, g2 * fmaf(u1, k1q2, g1 * b1));
                }
            }
            for (; t < nt; t++) {
                // Both products with the state as the last token left it, S: with S' = g S + k u^T the read-out is
                // S'^T q = g S^T q + u (k . q), so one exchange among a column's threads serves the write and the read-out.
                const float g = g_s[t], beta = g_s[ck + t], kq = g_s[2 * ck + t];
                const float v = col < Ps ? v_s[t * Ps + col] : 0.f;
                const float* kt = k_s + t * NP + part;
                const float* qt = q_s + t * NP + part;
                float kk[NPT];
                float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                for (int k = 0; k < NPT; k++) {
                    kk[k] = kt[k * parts];
                    const float qq = qt[k * parts];
                    if (k & 1) { a1 = fmaf(st[k], kk[k], a1); b1 = fmaf(st[k], qq, b1); }
                    else { a0 = fmaf(st[k], kk[k], a0); b0 = fmaf(st[k], qq, b0); }
                }
                float sk = a0 + a1, sq = b0 + b1;
                mm_parts_sum2(sk, sq, parts);
                const float uu = beta * (v - g * sk);
#pragma unroll
                for (int k = 0; k < NPT; k++) st[k] = fmaf(kk[k], uu, g * st[k]);
                if (live && part == 0) y[(size_t)(s.first + t0 + t) * H * E + h * E + e] = fmaf(uu, kq, g * sq);
            }
        }
        __syncthreads();
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

// The matrix LSTM's recurrence has no product with the state ahead of the write, so a column's threads need not meet token by
// token.  grid (segments, heads, slices of e); thread (col, part) = (tid % Ps, tid / Ps) of the first Ps * parts threads holds
// rows part NPT ... part NPT + NPT - 1 of column p0 + col; each leaves its share of S'^T q in shared memory and a chunk's
// shares are added afterwards, in the order of the parts.  The normaliser n is one column more, whose value is always one: the
// warp behind them holds it (its first `parts` threads), in a head's first slice only, which writes n' . q and exp(-m') a token
// and head to dn; the division waits for the kernel behind this one.  The last MM_FETCHERS threads fetch the NEXT chunk
// meanwhile (two buffers) and turn its gates into the three factors of a token, the running maximum going from token to token.
// u: [tokens, u_width] of the compute dtype, q at 0 (H d), k at H d, v at 2 H d (H e).  gates: [tokens, 2 H] float, i_raw | f_raw.
#define MM_FETCHERS (32 + MM_LOADERS)      // a warp for the gates, the others for keys, queries and values
#define MM_SCAN_THREADS (256 + 32 + MM_FETCHERS)
template <typename T, int NPT>
__global__ void __launch_bounds__(MM_SCAN_THREADS, 1) mlstm_scan_kernel(const T* __restrict__ u, int u_width, const float* __restrict__ gates,
                                                                    const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                                                                    float cap, const MMSegment* __restrict__ segs, float* state,
                                                                    long long state_stride, float* __restrict__ nm_buf,
                                                                    float* __restrict__ y, float* __restrict__ dn, int H, int d, int E,
                                                                    int Ps, int parts, int ck) {
    extern __shared__ __align__(16) float mm_smem[];
    constexpr int VEC = MMVec<T>::N;
    const int NP = NPT * parts, C = Ps + 1;
    // a buffer: q [ck][NP] | k [ck][NP] | v [ck][Ps] | exp(f + m - m') [ck] | exp(i - m') [ck] | exp(-m') [ck]
    const int BUF = ck * (2 * NP + Ps + 3);
    float* y_s = mm_smem + 2 * BUF;              // [ck][parts][C]
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, p0 = blockIdx.z * Ps;
    const int tid = threadIdx.x;
    const int main_threads = Ps * parts, fetch0 = (int)blockDim.x - MM_FETCHERS, side0 = fetch0 - 32;
    const bool fetcher = tid >= fetch0;
    const int ft = tid - fetch0, lane = tid & 31;
    const bool side = !fetcher && tid >= side0;                               // a thread of the normaliser's column
    const int col = side ? Ps : tid % Ps, part = side ? tid - side0 : tid / Ps;
    const bool active = side ? (blockIdx.z == 0 && part < parts) : tid < main_threads;
    const int e = p0 + col;
    float* slot = state + (size_t)s.slot * state_stride;
    float* S = slot + (size_t)h * d * E;
    const float* n_st = slot + (size_t)H * d * E + (size_t)h * d;
    float st[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part * NPT + k;
        float x = 0.f;
        if (active && n < d && s.before > 0) {
            if (side) x = n_st[n];
            else if (e < E) x = S[(size_t)n * E + e];
        }
        st[k] = x;
    }
    float m = s.before > 0 ? slot[(size_t)H * d * E + (size_t)H * d + h] : 0.f;        // (the fetchers' first warp's)
    const float bi = i_bias[h], bf = f_bias[h];
    const float q_scale = rsqrtf((float)d);
    const bool vec = d % VEC == 0 && u_width % VEC == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0;
    if (NP > d) {                                   // (the padding rows stay zero)
        for (int b = 0; b < 2; b++)
            for (int i = tid; i < 2 * ck * NP; i += blockDim.x) mm_smem[b * BUF + i] = 0.f;
        __syncthreads();
    }
    const int n_chunks = (s.count + ck - 1) / ck;
    for (int cc = -1; cc < n_chunks; cc++) {
        if (fetcher) {
            if (cc + 1 < n_chunks) {
                const int t0 = (cc + 1) * ck, nt = min(ck, s.count - t0);
                float* q_s = mm_smem + ((cc + 1) & 1) * BUF;
                float* k_s = q_s + ck * NP;
                float* v_s = k_s + ck * NP;
                float* a_s = v_s + ck * Ps;
                // every load of the chunk leaves before the first one is waited for: the values' first rounds, then keys
                // and queries
                if (ft >= 32) {
                const int fl = ft - 32;
                float rv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = fl + j * MM_LOADERS, ee = p0 + i % Ps;
                    rv[j] = (i < nt * Ps && ee < E) ? to_f32(u[(size_t)(s.first + t0 + i / Ps) * u_width + 2 * H * d + h * E + ee]) : 0.f;
                }
                if (vec) {
                    const int dv = d / VEC;
#pragma unroll 4
                    for (int i = fl; i < nt * dv; i += MM_LOADERS) {
                        const int t = i / dv, j = (i - t * dv) * VEC;
                        const T* row = u + (size_t)(s.first + t0 + t) * u_width + h * d + j;
                        mm_fetch16(row, q_s + t * NP + j, q_scale);
                        mm_fetch16(row + (size_t)H * d, k_s + t * NP + j, 1.f);
                    }
                } else {
                    for (int i = fl; i < nt * d; i += MM_LOADERS) {
                        const T* row = u + (size_t)(s.first + t0 + i / d) * u_width + h * d + i % d;
                        q_s[(i / d) * NP + i % d] = to_f32(row[0]) * q_scale;
                        k_s[(i / d) * NP + i % d] = to_f32(row[(size_t)H * d]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = fl + j * MM_LOADERS;
                    if (i < nt * Ps) v_s[i] = rv[j];
                }
#pragma unroll 4
                for (int i = fl + 4 * MM_LOADERS; i < nt * Ps; i += MM_LOADERS) {
                    const int ee = p0 + i % Ps;
                    v_s[i] = ee < E ? to_f32(u[(size_t)(s.first + t0 + i / Ps) * u_width + 2 * H * d + h * E + ee]) : 0.f;
                }
                } else {
                    // the fetchers' first warp: lane t has token t's gates; the running maximum goes from token to token,
                    // every lane following it
                    float fg = 0.f, ig = 0.f;
                    if (lane < nt) {
                        const float* r = gates + (size_t)(s.first + t0 + lane) * 2 * H;
                        fg = mm_logsigmoid(cap * tanhf((r[H + h] + bf) / cap));
                        ig = cap * tanhf((r[h] + bi) / cap);
                    }
                    float m_old = 0.f, m_new = 0.f;
                    for (int t = 0; t < nt; t++) {
                        const float fgt = __shfl_sync(0xffffffffu, fg, t), igt = __shfl_sync(0xffffffffu, ig, t);
                        const float mn = fmaxf(fgt + m, igt);
                        if (lane == t) { m_old = m; m_new = mn; }
                        m = mn;
                    }
                    if (lane < nt) {
                        a_s[lane] = expf(fg + m_old - m_new);
                        a_s[ck + lane] = expf(ig - m_new);
                        a_s[2 * ck + lane] = expf(-m_new);
                    }
                }
            }
        } else if (cc >= 0 && active) {
            const int nt = min(ck, s.count - cc * ck);
            const float* q_s = mm_smem + (cc & 1) * BUF;
            const float* k_s = q_s + ck * NP;
            const float* v_s = k_s + ck * NP;
            const float* a_s = v_s + ck * Ps;
#pragma unroll 2
            for (int t = 0; t < nt; t++) {
                const float a = a_s[t], b = a_s[ck + t];
                const float bv = side ? b : b * v_s[t * Ps + col];
                const float4* k4 = reinterpret_cast<const float4*>(k_s + t * NP + part * NPT);
                const float4* q4 = reinterpret_cast<const float4*>(q_s + t * NP + part * NPT);
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int k = 0; k < NPT / 4; k++) {
                    const float4 kv = k4[k], qv = q4[k];
                    st[4 * k + 0] = fmaf(a, st[4 * k + 0], kv.x * bv); acc0 = fmaf(st[4 * k + 0], qv.x, acc0);
                    st[4 * k + 1] = fmaf(a, st[4 * k + 1], kv.y * bv); acc1 = fmaf(st[4 * k + 1], qv.y, acc1);
                    st[4 * k + 2] = fmaf(a, st[4 * k + 2], kv.z * bv); acc0 = fmaf(st[4 * k + 2], qv.z, acc0);
                    st[4 * k + 3] = fmaf(a, st[4 * k + 3], kv.w * bv); acc1 = fmaf(st[4 * k + 3], qv.w, acc1);
                }
                y_s[(t * parts + part) * C + col] = acc0 + acc1;
            }
        }
        __syncthreads();
        if (cc >= 0) {
            const int t0 = cc * ck, nt = min(ck, s.count - t0);
            const float* em_s = mm_smem + (cc & 1) * BUF + ck * (2 * NP + Ps + 2);
            for (int i = tid; i < nt * C; i += blockDim.x) {
                const int t = i / C, c1 = i - t * C;
                if (c1 == Ps ? blockIdx.z != 0 : p0 + c1 >= E) continue;
                float acc = 0.f;
                for (int q = 0; q < parts; q++) acc += y_s[(t * parts + q) * C + c1];          // always in the order of the parts
                const size_t tok = (size_t)(s.first + t0 + t);
                if (c1 < Ps) y[tok * H * E + h * E + p0 + c1] = acc;
                else { dn[(tok * H + h) * 2] = acc; dn[(tok * H + h) * 2 + 1] = em_s[t]; }
            }
            __syncthreads();
        }
    }
    // Every slice of a head reads the head's m when it starts, and slices start at different times: the new n and m go to a
    // scratch row of the step, and the kernel behind this one moves them into the slot.
    float* nm = nm_buf + ((size_t)blockIdx.x * H + h) * (d + 1);
    if (active) {
#pragma unroll
        for (int k = 0; k < NPT; k++) {
            const int n = part * NPT + k;
            if (n < d) {
                if (side) nm[n] = st[k];
                else if (e < E) S[(size_t)n * E + e] = st[k];
            }
        }
    }
    if (blockIdx.z == 0 && ft == 0) nm[d] = m;
}

// The same for a step of decoded tokens, whose CTAs are many and short: every thread fetches, then the recurrence, then the
// shares are added; fewer threads and registers, more CTAs an SM.
#define MM_STEP_THREADS 288
template <typename T, int NPT>
__global__ void __launch_bounds__(MM_STEP_THREADS) mlstm_step_kernel(const T* __restrict__ u, int u_width, const float* __restrict__ gates,
                                                                    const float* __restrict__ i_bias, const float* __restrict__ f_bias,
                                                                    float cap, const MMSegment* __restrict__ segs, float* state,
                                                                    long long state_stride, float* __restrict__ nm_buf,
                                                                    float* __restrict__ y, float* __restrict__ dn, int H, int d, int E,
                                                                    int Ps, int parts, int ck) {
    extern __shared__ __align__(16) float mm_smem[];
    constexpr int VEC = MMVec<T>::N;
    const int NP = NPT * parts, C = Ps + 1;
    float* q_s = mm_smem;                        // [ck][NP]
    float* k_s = q_s + ck * NP;                  // [ck][NP]
    float* v_s = k_s + ck * NP;                  // [ck][Ps]
    float* a_s = v_s + ck * Ps;                  // [ck] exp(f + m - m') | [ck] exp(i - m') | [ck] exp(-m')
    float* y_s = a_s + 3 * ck;                   // [ck][parts][C]
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const MMSegment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, p0 = blockIdx.z * Ps;
    const int tid = threadIdx.x, lane = tid & 31;
    const int main_threads = Ps * parts, side0 = (int)blockDim.x - 32;
    const bool side = tid >= side0;                                           // a thread of the normaliser's column
    const int col = side ? Ps : tid % Ps, part = side ? tid - side0 : tid / Ps;
    const bool active = side ? (blockIdx.z == 0 && part < parts) : tid < main_threads;
    const int e = p0 + col;
    float* slot = state + (size_t)s.slot * state_stride;
    float* S = slot + (size_t)h * d * E;
    const float* n_st = slot + (size_t)H * d * E + (size_t)h * d;
    float st[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part * NPT + k;
        float x = 0.f;
        if (active && n < d && s.before > 0) {
            if (side) x = n_st[n];
            else if (e < E) x = S[(size_t)n * E + e];
        }
        st[k] = x;
    }
    float m = s.before > 0 ? slot[(size_t)H * d * E + (size_t)H * d + h] : 0.f;        // (the first warp's)
    const float bi = i_bias[h], bf = f_bias[h];
    const float q_scale = rsqrtf((float)d);
    const bool vec = d % VEC == 0 && u_width % VEC == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0;
    if (NP > d) for (int i = tid; i < 2 * ck * NP; i += blockDim.x) q_s[i] = 0.f;      // (the padding rows stay zero)
    for (int t0 = 0; t0 < s.count; t0 += ck) {
        const int nt = min(ck, s.count - t0);
        __syncthreads();
        if (vec) {
            const int dv = d / VEC;
#pragma unroll 2
            for (int i = tid; i < nt * dv; i += blockDim.x) {
                const int t = i / dv, j = (i - t * dv) * VEC;
                const T* row = u + (size_t)(s.first + t0 + t) * u_width + h * d + j;
                mm_fetch16(row, q_s + t * NP + j, q_scale);
                mm_fetch16(row + (size_t)H * d, k_s + t * NP + j, 1.f);
            }
        } else {
            for (int i = tid; i < nt * d; i += blockDim.x) {
                const T* row = u + (size_t)(s.first + t0 + i / d) * u_width + h * d + i % d;
                q_s[(i / d) * NP + i % d] = to_f32(row[0]) * q_scale;
                k_s[(i / d) * NP + i % d] = to_f32(row[(size_t)H * d]);
            }
        }
        for (int i = tid; i < nt * Ps; i += blockDim.x) {
            const int ee = p0 + i % Ps;
            v_s[i] = ee < E ? to_f32(u[(size_t)(s.first + t0 + i / Ps) * u_width + 2 * H * d + h * E + ee]) : 0.f;
        }
        if (tid < 32) {
            // lane t has token t's gates; the running maximum goes from token to token, every lane following it
            float fg = 0.f, ig = 0.f;
            if (lane < nt) {
                const float* r = gates + (size_t)(s.first + t0 + lane) * 2 * H;
                fg = mm_logsigmoid(cap * tanhf((r[H + h] + bf) / cap));
                ig = cap * tanhf((r[h] + bi) / cap);
            }
            float m_old = 0.f, m_new = 0.f;
            for (int t = 0; t < nt; t++) {
                const float ft = __shfl_sync(0xffffffffu, fg, t), it = __shfl_sync(0xffffffffu, ig, t);
                const float mn = fmaxf(ft + m, it);
                if (lane == t) { m_old = m; m_new = mn; }
                m = mn;
            }
            if (lane < nt) {
                a_s[lane] = expf(fg + m_old - m_new);
                a_s[ck + lane] = expf(ig - m_new);
                a_s[2 * ck + lane] = expf(-m_new);
            }
        }
        __syncthreads();
        if (active) {
#pragma unroll 2
            for (int t = 0; t < nt; t++) {
                const float a = a_s[t], b = a_s[ck + t];
                const float bv = side ? b : b * v_s[t * Ps + col];
                const float4* k4 = reinterpret_cast<const float4*>(k_s + t * NP + part * NPT);
                const float4* q4 = reinterpret_cast<const float4*>(q_s + t * NP + part * NPT);
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int k = 0; k < NPT / 4; k++) {
                    const float4 kv = k4[k], qv = q4[k];
                    st[4 * k + 0] = fmaf(a, st[4 * k + 0], kv.x * bv); acc0 = fmaf(st[4 * k + 0], qv.x, acc0);
                    st[4 * k + 1] = fmaf(a, st[4 * k + 1], kv.y * bv); acc1 = fmaf(st[4 * k + 1], qv.y, acc1);
                    st[4 * k + 2] = fmaf(a, st[4 * k + 2], kv.z * bv); acc0 = fmaf(st[4 * k + 2], qv.z, acc0);
                    st[4 * k + 3] = fmaf(a, st[4 * k + 3], kv.w * bv); acc1 = fmaf(st[4 * k + 3], qv.w, acc1);
                }
                y_s[(t * parts + part) * C + col] = acc0 + acc1;
            }
        }
        __syncthreads();
        for (int i = tid; i < nt * C; i += blockDim.x) {
            const int t = i / C, cc = i - t * C;
            if (cc == Ps ? blockIdx.z != 0 : p0 + cc >= E) continue;
            float acc = 0.f;
            for (int q = 0; q < parts; q++) acc += y_s[(t * parts + q) * C + cc];          // always in the order of the parts
            const size_t tok = (size_t)(s.first + t0 + t);
            if (cc < Ps) y[tok * H * E + h * E + p0 + cc] = acc;
            else { dn[(tok * H + h) * 2] = acc; dn[(tok * H + h) * 2 + 1] = a_s[2 * ck + t]; }
        }
    }
    // Every slice of a head reads the head's m when it starts, and slices start at different times: the new n and m go to a
    // scratch row of the step, and the kernel behind this one moves them into the slot.
    float* nm = nm_buf + ((size_t)blockIdx.x * H + h) * (d + 1);
    if (active) {
#pragma unroll
        for (int k = 0; k < NPT; k++) {
            const int n = part * NPT + k;
            if (n < d) {
                if (side) nm[n] = st[k];
                else if (e < E) S[(size_t)n * E + e] = st[k];
            }
        }
    }
    if (blockIdx.z == 0 && tid == 0) nm[d] = m;
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
// gain_per_head: the gain has H e entries, else e entries shared by the heads; kind 0 sigmoid, 1 silu.  With dn ([tokens, H, 2]:
// the normaliser's product with the query, exp(-m)) y holds numerators, and o = y / (max(|n . q|, exp(-m)) + 1e-6).
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* y, const float* __restrict__ dn, const T* gate, int g_stride,
                                                             const float* __restrict__ gain, T* __restrict__ out, long long n_rows,
                                                             int H, int E, int gain_per_head, int kind, float eps) {
    pdl_launch_dependents();
    pdl_wait(KID_MATRIX_MEMORY);
    const int lane = threadIdx.x & 31;
    const long long r = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const long long t = r / H;
    const int h = (int)(r % H);
    const float* yr = y + r * E;
    const T* gr = gate + t * g_stride + (size_t)h * E;
    const float over = dn ? fmaxf(fabsf(dn[r * 2]), dn[r * 2 + 1]) + 1e-6f : 1.0f;
    float ss = 0.f;
    for (int i = lane; i < E; i += 32) { const float v = yr[i] / over; ss += v * v; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps);
    for (int i = lane; i < E; i += 32) {
        const float z = to_f32(gr[i]);
        const float sg = mm_sigmoid(z);
        out[r * E + i] = from_f32<T>(yr[i] / over * inv * gain[gain_per_head ? h * E + i : i] * (kind == 1 ? z * sg : sg));
    }
}

struct MMShape { int parts, npt, Ps, slices, workers, threads, chunk; size_t smem; };

// The delta rule: PARTS threads a column so that a thread holds at most 16 rows (32 for the longest keys), columns a CTA so
// that a CTA has some 128 threads of state, fewer where that puts the step on more SMs.  Steps of decoded tokens fetch few
// tokens at a time: less shared memory, more CTAs an SM.
static inline int mm_shape(int n_segs, int H, int d, int E, int extra_floats, int max_segment_tokens, MMShape* out) {
    int parts = 1;
    while (parts < 32 && (d + parts - 1) / parts > 16) parts *= 2;
    const int rows = (d + parts - 1) / parts;
    if (rows > 32) return PLLM_ERR_LIMIT;
    const int npt = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    int Ps = 1;
    while (Ps * 2 * parts <= 128 && Ps < E) Ps *= 2;
    // (one CTA an SM, or a few more: two CTAs of a long recurrence on one SM take nearly twice as long)
    while (Ps * parts > 32 && (long long)n_segs * H * ((E + Ps - 1) / Ps) * 2 <= sm_count() + sm_count() / 8) Ps /= 2;
    out->parts = parts; out->npt = npt; out->Ps = Ps; out->slices = (E + Ps - 1) / Ps;
    out->workers = (Ps * parts + 31) / 32 * 32;
    const bool small = max_segment_tokens > 0 && max_segment_tokens <= MM_CHUNK_SMALL;
    out->threads = out->workers + (small ? MM_LOADERS_SMALL : MM_LOADERS);
    int chunk = small ? MM_CHUNK_SMALL : MM_CHUNK;
    auto smem_of = [&](int ck) { return 2 * (size_t)ck * (2 * npt * parts + Ps + extra_floats) * sizeof(float); };    // two buffers
    while (chunk > 4 && smem_of(chunk) > 72 * 1024) chunk /= 2;
    out->chunk = chunk;
    out->smem = smem_of(chunk);
    return out->smem > 200 * 1024 ? PLLM_ERR_LIMIT : PLLM_OK;
}

// The matrix LSTM: columns a CTA halved (down to 8) while the step's CTAs leave SMs empty, and while a thread would hold
// more than 16 rows; as many parts as 256 threads allow (32 at most: the normaliser's column is one warp), but no fewer
// than 4 rows a thread.
static inline int mlstm_shape(int n_segs, int H, int d, int E, int max_segment_tokens, MMShape* out) {
    int Ps = 1;
    while (Ps < E && Ps < 256) Ps *= 2;
    while (Ps > 8 && (long long)n_segs * H * ((E + Ps - 1) / Ps) * 2 <= sm_count() + sm_count() / 8) Ps /= 2;
    int parts, rows;
    for (;;) {
        parts = 256 / Ps > 32 ? 32 : 256 / Ps;
        while (parts > 1 && (parts / 2) * 4 >= d) parts /= 2;
        rows = (d + parts - 1) / parts;
        if (rows <= 16 || Ps <= 8) break;
        Ps /= 2;
    }
    if (rows > 32) return PLLM_ERR_LIMIT;
    const int npt = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    out->parts = parts; out->npt = npt; out->Ps = Ps; out->slices = (E + Ps - 1) / Ps;
    out->workers = (Ps * parts + 31) / 32 * 32;
    const bool small = max_segment_tokens > 0 && max_segment_tokens <= MM_CHUNK_SMALL;
    out->threads = out->workers + 32 + (small ? 0 : MM_FETCHERS);
    int chunk = small ? MM_CHUNK_SMALL : MM_CHUNK;
    auto smem_of = [&](int ck) { return (size_t)ck * ((small ? 1 : 2) * (2 * npt * parts + Ps + 3) + parts * (Ps + 1)) * sizeof(float); };   // buffers and the shares
    while (chunk > 4 && smem_of(chunk) > 128 * 1024) chunk /= 2;
    out->chunk = chunk;
    out->smem = smem_of(chunk);
    return (out->smem > 200 * 1024 || out->threads > MM_SCAN_THREADS) ? PLLM_ERR_LIMIT : PLLM_OK;
}

template <typename T>
static void launch_head_norm_gate(const float* y, const float* dn, const void* gate, int g_stride, const float* gain, void* out, int n_tokens, int H, int E,
                                  int gain_per_head, int kind, float eps, cudaStream_t stream) {
    const long long rows = (long long)n_tokens * H;
    launch_chained(head_norm_gate_kernel<T>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, stream, y, dn, (const T*)gate, g_stride, gain,
                   (T*)out, rows, H, E, gain_per_head, kind, eps);
}

#define MM_NPT_DISPATCH(npt, CALL) do { if ((npt) == 4) { constexpr int NPT = 4; CALL; } else if ((npt) == 8) { constexpr int NPT = 8; CALL; } \
    else if ((npt) == 16) { constexpr int NPT = 16; CALL; } else { constexpr int NPT = 32; CALL; } } while (0)

PLLM_EXPORT long long pllm_mlstm_state_floats(int H, int d, int E) { return (long long)H * d * E + (long long)H * d + H; }
PLLM_EXPORT long long pllm_delta_state_floats(int H, int G, int d, int E, int taps) {
    return (long long)H * d * E + (long long)(taps - 1) * (2 * G * d + H * E);
}

// u: [tokens, u_width] of the compute dtype: q (H d) | k (H d) | v (H e) | gate (H e); gates: [tokens, 2 H] float, i_raw | f_raw;
// gain: H e floats; nm_buf: [n_segs, H, d + 1], dn_buf: [tokens, H, 2] and y_buf: [tokens, H e] float scratch (rows of no
// segment zero in the last two); out: [tokens, H e] of the compute dtype.  max_segment_tokens bounds a segment's tokens (0: unknown).
PLLM_EXPORT int pllm_mlstm_mix(int dtype, const void* u, int u_width, const float* gates, const float* i_bias, const float* f_bias,
                               float cap, const float* gain, const int* segs, int n_segs, int max_segment_tokens, float* state,
                               long long state_stride, float* nm_buf, float* dn_buf, float* y_buf, void* out, int n_tokens, int H, int d,
                               int E, float eps, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return PLLM_OK;
    if (H <= 0 || d <= 0 || E <= 0 || !(cap > 0.f) || u_width < 2 * H * d + 2 * H * E) return PLLM_ERR_SIZE;
    if (state_stride < pllm_mlstm_state_floats(H, d, E)) return PLLM_ERR_SIZE;
    MMShape sh;
    const int rc = mlstm_shape(n_segs, H, d, E, max_segment_tokens, &sh);
    if (rc != PLLM_OK) return rc;
    PLLM_DISPATCH_DTYPE(dtype, {
        MM_NPT_DISPATCH(sh.npt, {
#define MM_MLSTM_SCAN(KERNEL) do { \
            if (sh.smem > 48 * 1024) cudaFuncSetAttribute(KERNEL<T, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh.smem); \
            launch_chained(KERNEL<T, NPT>, dim3(n_segs, H, sh.slices), dim3(sh.threads), sh.smem, stream, (const T*)u, u_width, \
                           gates, i_bias, f_bias, cap, (const MMSegment*)segs, state, state_stride, nm_buf, y_buf, dn_buf, H, d, E, sh.Ps, \
                           sh.parts, sh.chunk); } while (0)
            if (sh.threads == sh.workers + 32) MM_MLSTM_SCAN(mlstm_step_kernel); else MM_MLSTM_SCAN(mlstm_scan_kernel);
        });
        launch_chained(mlstm_store_nm_kernel, dim3(n_segs, H), dim3(128), 0, stream, (const float*)nm_buf, (const MMSegment*)segs, state,
                       state_stride, H, d, E);
        launch_head_norm_gate<T>(y_buf, dn_buf, (const T*)u + 2 * H * d + H * E, u_width, gain, out, n_tokens, H, E, 1, 0, eps, stream);
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
    const int rc = mm_shape(n_segs, H, d, E, 5, max_segment_tokens, &sh);
    if (rc != PLLM_OK) return rc;
    const int chunks = (max_segment_tokens + MM_CONV_TOKENS - 1) / MM_CONV_TOKENS;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(mm_conv_silu_kernel<T>, dim3(n_segs, (channels + 127) / 128, chunks > 0 ? chunks : 1), dim3(128), 0, stream,
                       (const T*)u, u_width, 0, (const T*)conv_w, (const MMSegment*)segs, (const float*)state, state_stride, conv_off,
                       c_buf, channels, taps);
#define MM_DELTA_SCAN(MINB) do { \
            if (sh.smem > 48 * 1024) \
                cudaFuncSetAttribute(delta_scan_kernel<T, NPT, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh.smem); \
            launch_chained(delta_scan_kernel<T, NPT, MINB>, dim3(n_segs, H, sh.slices), dim3(sh.threads), sh.smem, stream, (const float*)c_buf, \
                           channels, ba, (const T*)u, u_width, 0, a_log, dt_bias, (const MMSegment*)segs, state, state_stride, conv_off, \
                           y_buf, H, G, d, E, sh.Ps, sh.parts, taps, sh.chunk, sh.workers, sh.threads - sh.workers); } while (0)
        MM_NPT_DISPATCH(sh.npt, {
            if (sh.npt <= 16 && (long long)n_segs * H * sh.slices > sm_count()) MM_DELTA_SCAN(2); else MM_DELTA_SCAN(1);
        });
        launch_head_norm_gate<T>(y_buf, nullptr, (const T*)u + channels, u_width, gain, out, n_tokens, H, E, 0, 1, eps, stream);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(matrix_memory)
