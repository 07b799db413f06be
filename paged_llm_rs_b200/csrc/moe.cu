// A mixture of gated feed-forward experts: the router, the experts for a few rows, and what surrounds the
// grouped tensor-core products for many rows (sorting the pairs by expert, gathering, combining).
//
// Router (all float): z = W_r h over every router output (experts with tensors first, identity
// experts last); s = softmax(z); choice = s + correction.  Outputs form `groups` equal groups of
// neighbours; a group's score is its largest choice score, and only outputs of the `keep` best groups
// can be chosen (the others count as minus infinity).  The `top` largest choice scores are chosen; a
// chosen output's weight is its s divided by the sum of the chosen s (+ 1e-20).  Equal scores go to
// the lower index.  A bias (one float a router output) may be added to z; with a bias and no correction the weights
// are the softmax over the chosen logits alone, whatever their size among all.  The router's matrix may carry `extra`
// further rows behind its outputs, whose products with h leave as they are (a gate of the shared expert, say).
//
// Experts, the weight-streaming form: a (token, chosen expert) pair is a row of its own; a warp
// forms a few output columns at a time from that expert's weight rows, so every weight row that a step
// touches is read once per pair from L2 / HBM and nothing is read for experts that nobody chose.
//   pair_glu:   act[pair, :] = glu(Wg_e h, Wu_e h)     (silu(g) * u, or another gated activation of common.cuh)
//   pair_down:  out[t, :] = sum_k w[t, k] * (Wd_e act[pair]  |  h[t] for an identity expert) (+ shared[t, :], times
//               sigmoid(shared_gate[t]) when the shared expert is gated)
// The right form for the few tokens of a decode step and for the float32 engine; many rows in bfloat16
// go to the grouped tensor-core product instead.
#include "common.cuh"

enum : int { KID_MOE = 60 };

#define MOE_MAX_OUTPUTS 1024
#define MOE_MAX_TOP 32
// how router logits become scores and weights (bits of `scoring`): a sigmoid of each logit instead of the softmax over
// all; the chosen scores themselves as weights instead of their shares of the chosen scores' sum
enum : int { MOE_SCORE_SIGMOID = 1, MOE_SCORE_RAW_WEIGHTS = 2 };

// Every lane brings its best (value, index); all leave with the warp's best, ties to the lower index.
__device__ __forceinline__ void warp_argmax(float& best, int& at) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) { best = ov; at = oi; }
    }
}

// TOK tokens a CTA of eight warps.  The tokens' rows lie in shared memory as floats; warp w forms the logits of router
// outputs w, w + 8, ... for all of the CTA's tokens from one pass over each router row (float4 loads); then warp k
// does the softmax, the groups and the choice for token k.  h in T (the float32 engine's h is float); router weights
// and correction float.
template <typename T, int TOK>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* h, const float* __restrict__ w_router,
                                                        const float* __restrict__ correction, int* __restrict__ ids,
                                                        float* __restrict__ weights, int n_tokens, int width, int outputs,
                                                        int top, int groups, int keep, const float* __restrict__ bias, int extra,
                                                        float* __restrict__ extra_out, int scoring) {
    extern __shared__ float smem[];      // xs[TOK][width]; per token: s[outputs], choice[outputs], gscore[groups]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.x * TOK;
    float* xs = smem;
    float* per_token = xs + (size_t)TOK * width;
    const int per = 2 * outputs + groups + extra;
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    constexpr int N = Vec16<T>::N;
    if (width % N == 0) {
        for (int i = threadIdx.x * N; i < TOK * width; i += blockDim.x * N) {
            const int t = t0 + i / width;
            if (t < n_tokens) { Vec16<T> v; v.load(h + (size_t)t * width + i % width); v.unpack(xs + i); }
            else {
#pragma unroll
                for (int k = 0; k < N; k++) xs[i + k] = 0.f;
            }
        }
    } else {
        for (int i = threadIdx.x; i < TOK * width; i += blockDim.x) {
            const int t = t0 + i / width;
            xs[i] = t < n_tokens ? to_f32(h[(size_t)t * width + i % width]) : 0.f;
        }
    }
    __syncthreads();
    for (int e = warp; e < outputs + extra; e += 8) {
        const float* wr = w_router + (size_t)e * width;
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; k++) acc[k] = 0.f;
        if (width % 4 == 0) {
#pragma unroll 8
            for (int c = lane * 4; c < width; c += 128) {
                const float4 r = *reinterpret_cast<const float4*>(wr + c);
#pragma unroll
                for (int k = 0; k < TOK; k++) {
                    const float4 x = *reinterpret_cast<const float4*>(xs + k * width + c);
                    acc[k] = fmaf(x.x, r.x, fmaf(x.y, r.y, fmaf(x.z, r.z, fmaf(x.w, r.w, acc[k]))));
                }
            }
        } else {
            for (int c = lane; c < width; c += 32) {
                const float r = wr[c];
#pragma unroll
                for (int k = 0; k < TOK; k++) acc[k] = fmaf(xs[k * width + c], r, acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < TOK; k++) {
            const float z = warp_sum(acc[k]);
            if (lane == 0) {
                if (e < outputs) per_token[k * per + e] = z + (bias ? bias[e] : 0.f);
                else per_token[k * per + 2 * outputs + groups + (e - outputs)] = z;
            }
        }
    }
    __syncthreads();
    for (int k = warp; k < TOK; k += 8) {
        const int t = t0 + k;
        if (t >= n_tokens) continue;
        float* s = per_token + k * per;
        float* choice = s + outputs;
        float* gscore = choice + outputs;
        if (lane < extra) extra_out[(size_t)t * extra + lane] = gscore[groups + lane];
        if (scoring & MOE_SCORE_SIGMOID) {
            for (int e = lane; e < outputs; e += 32) {
                const float p = 1.0f / (1.0f + expf(-s[e]));
                s[e] = p;
                choice[e] = p + (correction ? correction[e] : 0.f);
            }
        } else {
            float zmax = -CUDART_INF_F;
            for (int e = lane; e < outputs; e += 32) zmax = fmaxf(zmax, s[e]);
            zmax = warp_max(zmax);
            float sum = 0.f;
            for (int e = lane; e < outputs; e += 32) { const float p = expf(s[e] - zmax); s[e] = p; sum += p; }
            sum = warp_sum(sum);
            __syncwarp();
            for (int e = lane; e < outputs; e += 32) {
                const float p = s[e] / sum;
                s[e] = p;
                choice[e] = p + (correction ? correction[e] : 0.f);
            }
        }
        __syncwarp();
        // groups: keep the best `keep`, the others' outputs cannot be chosen
        if (groups > 1 && keep < groups) {
            const int gsize = outputs / groups;
            for (int g = lane; g < groups; g += 32) {
                float gs = -CUDART_INF_F;
                for (int j = 0; j < gsize; j++) gs = fmaxf(gs, choice[g * gsize + j]);
                gscore[g] = gs;
            }
            __syncwarp();
            for (int round = 0; round < keep; round++) {
                float best = -CUDART_INF_F; int at = 0x7fffffff;
                for (int g = lane; g < groups; g += 32) {
                    const float gs = gscore[g];                    // (a kept group holds NaN and compares false)
                    if (gs > best || (gs == best && g < at)) { best = gs; at = g; }
                }
                warp_argmax(best, at);
                __syncwarp();
                if (lane == 0 && at != 0x7fffffff) gscore[at] = CUDART_NAN_F;
                __syncwarp();
            }
            for (int e = lane; e < outputs; e += 32)
                if (!isnan(gscore[e / gsize])) choice[e] = -CUDART_INF_F;
            __syncwarp();
        }
        // the `top` best choice scores
        float wsum = 0.f;
        int mine_id = 0; float mine_s = 0.f;      // lane j holds the j-th choice (top <= 32)
        for (int j = 0; j < top; j++) {
            float best = -CUDART_INF_F; int at = 0x7fffffff;
            for (int e = lane; e < outputs; e += 32) {
                const float c = choice[e];
                if (c > best) { best = c; at = e; }
            }
            warp_argmax(best, at);
            if (at == 0x7fffffff) at = 0;          // (cannot happen for a valid configuration)
            const float p = s[at];
            wsum += p;
            if (lane == j) { mine_id = at; mine_s = p; }
            __syncwarp();
            if (lane == 0) choice[at] = -CUDART_INF_F;
            __syncwarp();
        }
        if (lane < top) {
            ids[(size_t)t * top + lane] = mine_id;
            weights[(size_t)t * top + lane] = (scoring & MOE_SCORE_RAW_WEIGHTS) ? mine_s : mine_s / (wsum + 1e-20f);
        }
    }
}

template <typename T, int TOK>
static void launch_route(const void* h, const float* w_router, const float* correction, int* ids, float* weights, int n_tokens,
                         int width, int outputs, int top, int groups, int keep, const float* bias, int extra, float* extra_out,
                         int scoring, cudaStream_t stream) {
    const size_t smem = ((size_t)TOK * width + (size_t)TOK * (2 * outputs + groups + extra)) * sizeof(float);
    cudaFuncSetAttribute(moe_route_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(moe_route_kernel<T, TOK>, dim3((n_tokens + TOK - 1) / TOK), dim3(256), smem, stream, (const T*)h, w_router,
                   correction, ids, weights, n_tokens, width, outputs, top, groups, keep, bias, extra, extra_out, scoring);
}

// bias: [outputs] or null.  extra (<= 32): rows of w_router behind the outputs; extra_out [tokens, extra] receives their products.
PLLM_EXPORT int pllm_moe_route(int dtype, const void* h, const float* w_router, const float* correction, int* ids, float* weights,
                               int n_tokens, int width, int outputs, int top, int groups, int keep, const float* bias, int extra,
                               float* extra_out, int scoring, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (scoring < 0 || scoring > 3) return PLLM_ERR_SIZE;
    if (extra < 0 || extra > 32 || (extra > 0 && !extra_out)) return PLLM_ERR_SIZE;
    if (width <= 0 || outputs <= 0 || top <= 0 || groups <= 0 || keep <= 0 || outputs % groups || keep > groups) return PLLM_ERR_SIZE;
    if (outputs > MOE_MAX_OUTPUTS || top > MOE_MAX_TOP || top > outputs) return PLLM_ERR_LIMIT;
    // eight tokens a CTA from some hundreds of tokens on (a router row is then read once for the eight), where they fit
    const bool many = n_tokens >= 256 && (8 * (size_t)width + 8 * (size_t)(2 * outputs + groups + extra)) * sizeof(float) <= 160 * 1024;
    if (((size_t)width + 2 * outputs + groups + extra) * sizeof(float) > 200 * 1024) return PLLM_ERR_LIMIT;
    PLLM_DISPATCH_DTYPE(dtype, {
        if (many) launch_route<T, 8>(h, w_router, correction, ids, weights, n_tokens, width, outputs, top, groups, keep, bias, extra, extra_out, scoring, stream);
        else launch_route<T, 1>(h, w_router, correction, ids, weights, n_tokens, width, outputs, top, groups, keep, bias, extra, extra_out, scoring, stream);
    });
    return launch_status();
}

// ---- the experts for a few rows -----------------------------------------------------------------
// w_gu: [experts, 2 * ff, width] (an expert's gate rows, then its up rows); act: [pairs, ff].
// grid (pairs, column blocks); a CTA keeps the token's row in shared memory as floats; a warp forms PAIR_CW columns
// at a time, so that the loads of 2 * PAIR_CW weight rows are in flight together.
#define PAIR_CW 4
// GATED false: the experts have no gate rows (w_gu is [experts, ff, width]) and `glu` names a one-argument activation
// (common.cuh: UNARY_*).  in_weights [pairs] or null: the expert reads the token times the pair's weight, which is the weight
// times the products with the token itself.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_pair_glu_kernel(const T* h, const int* ids, const T* __restrict__ w_gu, T* __restrict__ act,
                                                           int width, int ff, int top, int experts, int glu, float limit,
                                                           const float* __restrict__ in_weights) {
    extern __shared__ float xs[];
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    const int e = ids[pair];
    if (e < 0 || e >= experts) return;             // an identity expert has no product
    constexpr int N = Vec16<T>::N;
    const bool vec = width % N == 0;
    const T* hr = h + (size_t)(pair / top) * width;
    if (vec) {
        for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) { Vec16<T> v; v.load(hr + c); v.unpack(xs + c); }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32(hr[c]);
    }
    __syncthreads();
    const T* wg = w_gu + (size_t)e * (GATED ? 2 : 1) * ff * width;
    const T* wu = GATED ? wg + (size_t)ff * width : wg;
    const float in_w = in_weights ? in_weights[pair] : 1.0f;
    const int col0 = (blockIdx.y * 8 + warp) * PAIR_CW;
    if (col0 >= ff) return;
    float ag[PAIR_CW], au[PAIR_CW];
#pragma unroll
    for (int j = 0; j < PAIR_CW; j++) { ag[j] = 0.f; au[j] = 0.f; }
    if (vec) {
#pragma unroll 2
        for (int c = lane * N; c < width; c += 32 * N) {
            Vec16<T> vg[PAIR_CW], vu[PAIR_CW];
#pragma unroll
            for (int j = 0; j < PAIR_CW; j++) {
                const int col = min(col0 + j, ff - 1);           // (a column past the end repeats the last one and is not stored)
                if (GATED) vg[j].load(wg + (size_t)col * width + c);
                vu[j].load(wu + (size_t)col * width + c);
            }
#pragma unroll
            for (int j = 0; j < PAIR_CW; j++) {
                float fg[N], fu[N];
                if (GATED) vg[j].unpack(fg);
                vu[j].unpack(fu);
#pragma unroll
                for (int k = 0; k < N; k++) {
                    if (GATED) ag[j] = fmaf(xs[c + k], fg[k], ag[j]);
                    au[j] = fmaf(xs[c + k], fu[k], au[j]);
                }
            }
        }
    } else {
        for (int c = lane; c < width; c += 32) {
#pragma unroll
            for (int j = 0; j < PAIR_CW; j++) {
                const int col = min(col0 + j, ff - 1);
                if (GATED) ag[j] = fmaf(xs[c], to_f32(wg[(size_t)col * width + c]), ag[j]);
                au[j] = fmaf(xs[c], to_f32(wu[(size_t)col * width + c]), au[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < PAIR_CW; j++) {
        const float g = GATED ? warp_sum(ag[j]) * in_w : 0.f, u = warp_sum(au[j]) * in_w;
        if (lane == 0 && col0 + j < ff)
            act[(size_t)pair * ff + col0 + j] = from_f32<T>(GATED ? glu_act(glu, limit, g, u) : unary_act(glu, u));
    }
}

// w_d: [experts, width, ff].  grid (tokens, column blocks); a warp forms `cw` (1 or 2) columns.  The token's activations
// lie in shared memory already multiplied by their experts' weights, so a column is ONE sum over all chosen experts'
// rows (their loads in flight together) and one reduction.  shared: [tokens, width] or null.
template <typename T, int CW>
__global__ void __launch_bounds__(256) moe_pair_down_kernel(const T* act, const T* h, const int* ids, const float* weights,
                                                            const T* __restrict__ w_d, const T* shared, T* __restrict__ out,
                                                            int width, int ff, int top, int experts, const float* shared_gate,
                                                            int unit_weights) {
    extern __shared__ float xs[];                 // [top][ff]: weight_k * activation of expert k (zeros for an identity expert)
    __shared__ int id_s[MOE_MAX_TOP];
    __shared__ float idw_s;                       // the identity experts' weights, summed
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    if (threadIdx.x < 32) {
        int e = -1; float w = 0.f;
        if (lane < top) { e = ids[(size_t)t * top + lane]; w = weights[(size_t)t * top + lane]; }     // (an identity expert's weight counts either way)
        const bool identity = lane < top && (e < 0 || e >= experts);
        if (lane < top) id_s[lane] = identity ? -1 : e;
        const float iw = warp_sum(identity ? w : 0.f);
        if (lane == 0) idw_s = iw;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) {
        const int k = i / ff;
        xs[i] = id_s[k] < 0 ? 0.f : (unit_weights ? 1.0f : weights[(size_t)t * top + k]) * to_f32(act[((size_t)t * top + k) * ff + i % ff]);
    }
    __syncthreads();
    constexpr int N = Vec16<T>::N;
    const bool vec = ff % N == 0;
    const int col0 = (blockIdx.y * 8 + warp) * CW;
    if (col0 >= width) return;
    float acc[CW];
#pragma unroll
    for (int j = 0; j < CW; j++) acc[j] = 0.f;
    if (vec) {
        for (int c = lane * N; c < ff; c += 32 * N) {
#pragma unroll 4
            for (int k = 0; k < top; k++) {
                const int e = id_s[k];
                if (e < 0) continue;
                const float* x = xs + k * ff + c;
#pragma unroll
                for (int j = 0; j < CW; j++) {
                    const int col = min(col0 + j, width - 1);
                    Vec16<T> vd; vd.load(w_d + ((size_t)e * width + col) * ff + c);
                    float fd[N]; vd.unpack(fd);
#pragma unroll
                    for (int q = 0; q < N; q++) acc[j] = fmaf(x[q], fd[q], acc[j]);
                }
            }
        }
    } else {
        for (int k = 0; k < top; k++) {
            const int e = id_s[k];
            if (e < 0) continue;
#pragma unroll
            for (int j = 0; j < CW; j++) {
                const T* d = w_d + ((size_t)e * width + min(col0 + j, width - 1)) * ff;
                for (int c = lane; c < ff; c += 32) acc[j] = fmaf(xs[k * ff + c], to_f32(d[c]), acc[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CW; j++) {
        float total = warp_sum(acc[j]);
        const int col = col0 + j;
        if (lane == 0 && col < width) {
            if (idw_s != 0.f) total += idw_s * to_f32(h[(size_t)t * width + col]);      // identity experts: the input itself
            if (shared) total += to_f32(shared[(size_t)t * width + col]) * (shared_gate ? 1.0f / (1.0f + expf(-shared_gate[t])) : 1.0f);
            out[(size_t)t * width + col] = from_f32<T>(total);
        }
    }
}

// glu: a gated activation's kind (GLU_*), or with gated 0 a one-argument activation's (UNARY_*) for experts without gate rows.
PLLM_EXPORT int pllm_moe_pair_glu(int dtype, const void* h, const int* ids, const void* w_gu, void* act, int n_tokens, int width,
                                  int ff, int top, int experts, int glu, float limit, int gated, const float* in_weights,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (gated ? (glu < GLU_SILU || glu > GLU_CLAMPED) : (glu < UNARY_NONE || glu > UNARY_RELU2)) return PLLM_ERR_SIZE;
    if (width <= 0 || ff <= 0 || top <= 0 || experts <= 0) return PLLM_ERR_SIZE;
    if ((size_t)width * sizeof(float) > 200 * 1024) return PLLM_ERR_LIMIT;
    const dim3 grid(n_tokens * top, (ff + 8 * PAIR_CW - 1) / (8 * PAIR_CW));
    const size_t smem = (size_t)width * sizeof(float);
    PLLM_DISPATCH_DTYPE(dtype, {
        if (gated) {
            cudaFuncSetAttribute(moe_pair_glu_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_chained(moe_pair_glu_kernel<T, true>, grid, dim3(256), smem, stream, (const T*)h, ids, (const T*)w_gu, (T*)act, width,
                           ff, top, experts, glu, limit, in_weights);
        } else {
            cudaFuncSetAttribute(moe_pair_glu_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_chained(moe_pair_glu_kernel<T, false>, grid, dim3(256), smem, stream, (const T*)h, ids, (const T*)w_gu, (T*)act, width,
                           ff, top, experts, glu, limit, in_weights);
        }
    });
    return launch_status();
}

PLLM_EXPORT int pllm_moe_pair_down(int dtype, const void* act, const void* h, const int* ids, const float* weights, const void* w_d,
                                   const void* shared, void* out, int n_tokens, int width, int ff, int top, int experts,
                                   const float* shared_gate, int unit_weights, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (width <= 0 || ff <= 0 || top <= 0 || experts <= 0) return PLLM_ERR_SIZE;
    if (top > MOE_MAX_TOP) return PLLM_ERR_LIMIT;
    if ((size_t)top * ff * sizeof(float) > 200 * 1024) return PLLM_ERR_LIMIT;
    PLLM_DISPATCH_DTYPE(dtype, {
        cudaFuncSetAttribute(moe_pair_down_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)top * ff * sizeof(float)));
        cudaFuncSetAttribute(moe_pair_down_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)top * ff * sizeof(float)));
        // a column a warp while the tokens are few (every SM gets CTAs), two from a handful of tokens on
        if (n_tokens <= 4)
            launch_chained(moe_pair_down_kernel<T, 1>, dim3(n_tokens, (width + 7) / 8), dim3(256), (size_t)top * ff * sizeof(float),
                           stream, (const T*)act, (const T*)h, ids, weights, (const T*)w_d, (const T*)shared, (T*)out, width, ff, top,
                           experts, shared_gate, unit_weights);
        else
            launch_chained(moe_pair_down_kernel<T, 2>, dim3(n_tokens, (width + 15) / 16), dim3(256), (size_t)top * ff * sizeof(float),
                           stream, (const T*)act, (const T*)h, ids, weights, (const T*)w_d, (const T*)shared, (T*)out, width, ff, top,
                           experts, shared_gate, unit_weights);
    });
    return launch_status();
}

// ---- the experts for many rows: sort the pairs by expert, grouped tensor-core products, combine ----------------
// align:   slot_pair[slot] = pair or -1, pair_slot[pair] = slot or -1 (identity expert), tile_expert[tile] = expert or -1.
//          Expert e's pairs take consecutive slots from a multiple of 128 on; which pair gets which of them is
//          whatever order the atomics fall in, which changes no value: every row is multiplied on its own.
// gather:  xs[slot] = h[pair / top]  (zeros in the padding of a tile in use; tiles past the last are left alone)
// combine: out[t] = sum_k w[t, k] * (y[pair_slot] | h[t] for an identity expert) (+ shared[t])
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* ids, int n_pairs, int experts, int* __restrict__ slot_pair,
                                                         int* __restrict__ pair_slot, int* __restrict__ tile_expert, int max_tiles) {
    __shared__ int count[MOE_MAX_OUTPUTS], start[MOE_MAX_OUTPUTS];
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < max_tiles * 128; i += blockDim.x) slot_pair[i] = -1;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < experts; e++) {
            start[e] = tile * 128;
            const int tiles = (count[e] + 127) / 128;
            for (int k = 0; k < tiles && tile + k < max_tiles; k++) tile_expert[tile + k] = e;
            tile += tiles;
            count[e] = 0;
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        int slot = -1;
        if (e >= 0 && e < experts) {
            slot = start[e] + atomicAdd(&count[e], 1);
            if (slot < max_tiles * 128) slot_pair[slot] = p; else slot = -1;
        }
        pair_slot[p] = slot;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_gather_kernel(const T* h, const int* slot_pair, const int* tile_expert, T* __restrict__ xs,
                                                         int n_slots, int width, int top, const float* __restrict__ in_weights) {
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    const int lane = threadIdx.x & 31, slot = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (slot >= n_slots || tile_expert[slot >> 7] < 0) return;
    const int pair = slot_pair[slot];
    T* dst = xs + (size_t)slot * width;
    constexpr int N = Vec16<T>::N;
    if (pair < 0) {
        for (int c = lane; c < width; c += 32) dst[c] = from_f32<T>(0.f);
        return;
    }
    const T* src = h + (size_t)(pair / top) * width;
    if (in_weights) {                      // the expert reads the token times the pair's weight
        const float w = in_weights[pair];
        for (int c = lane; c < width; c += 32) dst[c] = from_f32<T>(to_f32(src[c]) * w);
        return;
    }
    if (width % N == 0) {
        for (int c = lane * N; c < width; c += 32 * N) { Vec16<T> v; v.load(src + c); v.store(dst + c); }
    } else {
        for (int c = lane; c < width; c += 32) dst[c] = src[c];
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* y, const T* h, const int* pair_slot, const float* weights,
                                                          const T* shared, T* __restrict__ out, int width, int top,
                                                          const float* shared_gate, int unit_weights) {
    pdl_launch_dependents();
    pdl_wait(KID_MOE);
    const int t = blockIdx.x;
    const float sg = shared_gate ? 1.0f / (1.0f + expf(-shared_gate[t])) : 1.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = shared ? to_f32(shared[(size_t)t * width + c]) * sg : 0.f;
        for (int k = 0; k < top; k++) {
            const int slot = pair_slot[(size_t)t * top + k];
            const float v = slot < 0 ? to_f32(h[(size_t)t * width + c]) : to_f32(y[(size_t)slot * width + c]);
            total = fmaf((unit_weights && slot >= 0) ? 1.0f : weights[(size_t)t * top + k], v, total);
        }
        out[(size_t)t * width + c] = from_f32<T>(total);
    }
}

PLLM_EXPORT int pllm_moe_align(const int* ids, int n_pairs, int experts, int* slot_pair, int* pair_slot, int* tile_expert,
                               int max_tiles, cudaStream_t stream) {
    if (n_pairs <= 0) return PLLM_OK;
    if (experts <= 0 || max_tiles <= 0) return PLLM_ERR_SIZE;
    if (experts > MOE_MAX_OUTPUTS) return PLLM_ERR_LIMIT;
    launch_chained(moe_align_kernel, dim3(1), dim3(1024), 0, stream, ids, n_pairs, experts, slot_pair, pair_slot, tile_expert, max_tiles);
    return launch_status();
}

PLLM_EXPORT int pllm_moe_gather(int dtype, const void* h, const int* slot_pair, const int* tile_expert, void* xs, int n_slots,
                                int width, int top, const float* in_weights, cudaStream_t stream) {
    if (n_slots <= 0) return PLLM_OK;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(moe_gather_kernel<T>, dim3((n_slots + 7) / 8), dim3(256), 0, stream, (const T*)h, slot_pair, tile_expert,
                       (T*)xs, n_slots, width, top, in_weights);
    });
    return launch_status();
}

PLLM_EXPORT int pllm_moe_combine(int dtype, const void* y, const void* h, const int* pair_slot, const float* weights,
                                 const void* shared, void* out, int n_tokens, int width, int top, const float* shared_gate,
                                 int unit_weights, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(moe_combine_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)y, (const T*)h, pair_slot, weights,
                       (const T*)shared, (T*)out, width, top, shared_gate, unit_weights);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(moe)
