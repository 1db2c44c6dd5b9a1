// Routed experts (mixture of experts): router, grouping of tokens by expert, the experts' two products as
// grouped matrix products, and the weighted sum.  Nothing here depends on the host: a step with routed
// experts records into a CUDA graph like any other.
//
//   z = W_r h + b_r                                  (float32; h in the activation type)
//   chosen = the `top` largest z (the lower index first among equals); weight_j = softmax over the chosen z
//   y = sum_j weight_j * W_down[e_j] ( silu(W_gate[e_j] h) * (W_up[e_j] h) )
// or, for experts without a gate whose weight acts on their input (score mode 1: weight_j = sigmoid(z_j), not renormalised):
//   y = sum_j W_down[e_j] act( W_up[e_j] (weight_j h) ) = sum_j W_down[e_j] act( weight_j * (W_up[e_j] h) ),  act = relu^2 or silu
// (epilogue UP_ACT: the weight multiplies the float32 result of the up product, which is the product of the weighted input).
//
// moe_route_kernel     one block per token: z, the choice and the weights            -> idx, wgt [T, top]
// moe_group_kernel     one block: entries (token, j) counted and listed per expert   -> offsets [E+1], tile_start
//                      [E+1] (tiles of bm rows per expert, running), perm [T*top] (place in expert order -> entry)
// moe_gemm_*_kernel    one block per (64-row tile of one expert's entries, 64 output features): bfloat16 on
//                      mma.sync.m16n8k16 from cp.async double-buffered tiles, or any type on the CUDA cores
//                      (float32 models; widths that are no multiple of 8).  Epilogue GATE_UP: silu(gate) * up
//                      into act [T*top, ff] in expert order; epilogue DOWN: float32 rows into out2 at the
//                      entry's own place [T*top, width].
// moe_combine_kernel   y[t] = sum_j wgt[t, j] * out2[t*top + j] in float32           -> y [T, width]
#include "mma_helpers.cuh"

#define MOE_BM 64
#define MOE_BN 64

enum { MOE_GATE_UP = 0, MOE_DOWN = 1, MOE_UP_ACT = 2 };
enum { MOE_ACT_SILU = 0, MOE_ACT_RELU2 = 1, MOE_ACT_CAPPED = 2 };   // CAPPED (gated experts): see moe_glu
enum { MOE_SCORE_SOFTMAX_CHOSEN = 0, MOE_SCORE_SIGMOID = 1, MOE_SCORE_SOFTMAX_ALL = 2 };

// TOK tokens per block (their rows of h in shared memory as float32, so that a warp reads an expert's router row once
// for all of them); 8 warps take the experts in turn; warp w < TOK then chooses for token w.
template <typename TA, int TOK>
__global__ void __launch_bounds__(256) moe_route_kernel(const TA* __restrict__ h, const float* __restrict__ wr,
                                                        const float* __restrict__ br, int T, int D, int E, int top,
                                                        int mode, int* __restrict__ idx, float* __restrict__ wgt,
                                                        const float* __restrict__ choice_bias, float weight_scale,
                                                        int groups, int groups_keep, int renorm) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float rsm[];       // TOK rows of D floats (D rounded up to 4), then TOK x E logits (twice for mode 2)
    const int Dp = (D + 3) & ~3;
    float* hs = rsm;
    float* z = rsm + TOK * Dp;
    const int t0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int nt = min(TOK, T - t0);
#pragma unroll 4
    for (int i = threadIdx.x; i < TOK * D; i += blockDim.x) {
        const int k = i / D, d = i - k * D;
        hs[k * Dp + d] = k < nt ? to_f32(h[(size_t)(t0 + k) * D + d]) : 0.f;
    }
    __syncthreads();
    const bool vec = (D & 3) == 0;
    for (int e = warp; e < E; e += nw) {
        const float* w = wr + (size_t)e * D;
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) acc[k] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int i = lane * 4; i < D; i += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
                for (int k = 0; k < TOK; ++k) {
                    const float4 hv = *reinterpret_cast<const float4*>(hs + k * Dp + i);
                    acc[k] += (hv.x * wv.x + hv.y * wv.y) + (hv.z * wv.z + hv.w * wv.w);
                }
            }
        } else {
            for (int i = lane; i < D; i += 32) {
                const float wv = w[i];
#pragma unroll
                for (int k = 0; k < TOK; ++k) acc[k] += hs[k * Dp + i] * wv;
            }
        }
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            const float a = warp_sum(acc[k]);
            if (lane == 0) z[k * E + e] = a + (br ? br[e] : 0.f);
        }
    }
    __syncthreads();
    if (warp >= nt) return;
    float* zt = z + warp * E;
    const int t = t0 + warp;
    // mode 2: the score of an expert is its share of the softmax over ALL logits; the choice is by score + choice_bias, the
    // weight is the score itself (times weight_scale), not renormalised over the chosen
    float* score = z + TOK * E + warp * E;
    if (mode == MOE_SCORE_SOFTMAX_ALL) {
        float mx = -INFINITY, den = 0.f;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zt[e]);
        mx = warp_max(mx);
        for (int e = lane; e < E; e += 32) den += expf(zt[e] - mx);
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) {
            const float p = expf(zt[e] - mx) / den;
            score[e] = p;
            zt[e] = p + (choice_bias ? choice_bias[e] : 0.f);
        }
        __syncwarp();
        // groups of neighbouring experts: only the groups_keep groups whose best number (score + bias) is largest stay in
        // the choice (the lower group first among equals); the others count as minus infinity
        if (groups > 1 && groups_keep < groups) {
            float* gbest = z + 2 * TOK * E + warp * E;          // [groups], then which groups stay
            const int per = E / groups;
            for (int g = lane; g < groups; g += 32) {
                float b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, zt[e]);
                gbest[g] = b;
            }
            __syncwarp();
            for (int g = lane; g < groups; g += 32) {
                const float mine_b = gbest[g];
                int ahead = 0;                                   // groups that come before this one in the order
                for (int o = 0; o < groups; ++o) {
                    const float ob = gbest[o];
                    ahead += (ob > mine_b || (ob == mine_b && o < g)) ? 1 : 0;
                }
                if (ahead >= groups_keep)
                    for (int e = g * per; e < (g + 1) * per; ++e) zt[e] = -INFINITY;
            }
            __syncwarp();
        }
    }
    float first = 0.f, sum = 0.f, mine = 0.f;    // lane j keeps the j-th chosen logit (top <= 32)
    int mine_e = 0;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = zt[e];
            if (v > best || (v == best && e < be)) { best = v; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
        }
        if (be == 0x7fffffff) be = 0;           // only NaN or -inf left: keep indices legal
        if (j == 0) first = best;
        const float p = mode == MOE_SCORE_SOFTMAX_ALL ? score[be] * weight_scale
                        : mode == MOE_SCORE_SIGMOID ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
        sum += p;
        if (lane == j) { mine = p; mine_e = be; }
        __syncwarp();
        if (lane == 0) zt[be] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        idx[(size_t)t * top + lane] = mine_e;
        // renorm (softmax over all): the chosen scores divided by their sum; sum holds them times weight_scale
        wgt[(size_t)t * top + lane] = mode == MOE_SCORE_SOFTMAX_CHOSEN ? mine / sum
                                      : renorm ? mine / (sum / weight_scale + 1e-20f) : mine;
    }
}

// One block.  n entries (token-major: entry = t * top + j).
__global__ void moe_group_kernel(const int* __restrict__ idx, int n, int E, int bm, int* __restrict__ offsets,
                                 int* __restrict__ tile_start, int* __restrict__ perm, int* __restrict__ place) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int sm[];        // counts [E], starts [E]
    int* counts = sm;
    int* starts = sm + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            tile_start[e] = tiles;
            starts[e] = at;
            at += counts[e];
            tiles += (counts[e] + bm - 1) / bm;
        }
        offsets[E] = at;
        tile_start[E] = tiles;
    }
    __syncthreads();
    // the order of one expert's entries is left to the atomics: every row of a grouped product is computed by
    // itself, so the order changes no result
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int p = atomicAdd(&starts[idx[i]], 1);
        perm[p] = i;
        if (place) place[i] = p;
    }
}

__device__ __forceinline__ int moe_find_expert(const int* __restrict__ tile_start, int E, int tile) {
    int lo = 0, hi = E;                 // the largest e with tile_start[e] <= tile
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= tile) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float moe_silu(float g) { return g / (1.0f + expf(-g)); }
// What a gated expert makes of its gate and up products: silu(g) u, or with a cap L (MOE_ACT_CAPPED)
// g' sigmoid(1.702 g') (u' + 1) with g' = min(g, L) and u' = clamp(u, -L, L).
__device__ __forceinline__ float moe_glu(float g, float u, int act, float limit) {
    if (act == MOE_ACT_CAPPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return moe_silu(g) * u;
}
__device__ __forceinline__ float moe_act(float u, int act) {
    if (act == MOE_ACT_RELU2) { const float r = fmaxf(u, 0.f); return r * r; }
    return moe_silu(u);
}

// bfloat16 on tensor cores.  a: EPI GATE_UP: x [T, K] (row of entry p: perm[p] / top); EPI DOWN: act [n, K] in
// expert order.  w: [E, NW, K] with NW = 2 * N (gate rows, then up rows) or N.  K a multiple of 8.
// BM = 64: four warps take 16 rows each over all 64 features, two stages.  BM = 16 (a handful of tokens: an expert's
// list is short and the kernel is a stream of weights): the four warps split the 64 features, four stages, and the
// smaller block leaves room for four blocks per SM - three times the bytes in flight; the down product, whose blocks
// are few (width / 64 per expert) and hold one weight block a stage, takes 64 instead of 32 of K per stage.
template <int EPI, int BM, int BK>
__global__ void __launch_bounds__(128) moe_gemm_mma_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w,
                                                           const int* __restrict__ offsets,
                                                           const int* __restrict__ tile_start,
                                                           const int* __restrict__ perm, int E, int top, int N, int K,
                                                           bf16* __restrict__ act, float* __restrict__ out2,
                                                           const float* __restrict__ wgt, int act_kind, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NB = EPI == MOE_GATE_UP ? 2 : 1;
    constexpr int WM = BM / 16, WN = 4 / WM, NT = MOE_BN / WN / 8, ST = BM == 64 ? 2 : 4;
    constexpr int LD = BK + 8, CH = BK / 8;      // elements per shared-memory row (ldmatrix rows in distinct banks); 16-byte chunks per row
    __shared__ __align__(16) bf16 sa[ST][BM][LD];
    __shared__ __align__(16) bf16 sw[ST][NB][MOE_BN][LD];
    __shared__ int src_row[BM];
    const int tile = blockIdx.x;
    if (tile >= tile_start[E]) return;
    const int e = moe_find_expert(tile_start, E, tile);
    const int p0 = offsets[e] + (tile - tile_start[e]) * BM;
    const int nrows = min(BM, offsets[e + 1] - p0);
    const int n0 = blockIdx.y * MOE_BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row0 = (warp % WM) * 16, col0 = (warp / WM) * NT * 8;
    for (int r = tid; r < BM; r += 128)
        src_row[r] = r < nrows ? (EPI != MOE_DOWN ? perm[p0 + r] / top : p0 + r) : -1;
    __syncthreads();
    const bf16* we = w + (size_t)e * NB * N * K;

    auto load = [&](int stage, int k0) {
        // rows x CH chunks of 8 elements each for a, the same per weight block
        for (int c = tid; c < BM * CH; c += 128) {
            const int r = c / CH, kc = (c % CH) * 8;
            const int sr = src_row[r];
            const bool ok = sr >= 0 && k0 + kc < K;
            cp_async_16(smem_u32(&sa[stage][r][kc]), a + (size_t)(ok ? sr : 0) * K + (ok ? k0 + kc : 0), ok);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = tid; c < MOE_BN * CH; c += 128) {
                const int r = c / CH, kc = (c % CH) * 8;
                const bool ok = n0 + r < N && k0 + kc < K;
                cp_async_16(smem_u32(&sw[stage][b][r][kc]),
                            we + ((size_t)b * N + (ok ? n0 + r : 0)) * K + (ok ? k0 + kc : 0), ok);
            }
        cp_async_commit();
    };

    float acc[NB][NT][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[b][j][i] = 0.f;

    const int nk = (K + BK - 1) / BK;
#pragma unroll
    for (int s0 = 0; s0 < ST - 1; ++s0) {
        if (s0 < nk) load(s0, s0 * BK);
        else cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        const int st = kt % ST;
        cp_async_wait<ST - 2>();         // the copies of stage kt have landed
        __syncthreads();                 // ... for every thread, and everyone is done with stage kt - 1
        if (kt + ST - 1 < nk) load((kt + ST - 1) % ST, (kt + ST - 1) * BK);
        else cp_async_commit();
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t fa[4];
            ldmatrix_x4(fa, smem_u32(&sa[st][row0 + (lane & 15)][kk + (lane >> 4) * 8]));
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    uint32_t fb[4];
                    ldmatrix_x4(fb, smem_u32(&sw[st][b][col0 + j * 8 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]));
                    mma_bf16(acc[b][j], fa, fb[0], fb[1]);
                    mma_bf16(acc[b][j + 1], fa, fb[2], fb[3]);
                }
        }
    }
    // epilogue: a thread holds rows row0 + lane/4 (+8) and columns col0 + j*8 + (lane%4)*2 (+1)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = row0 + (lane >> 2) + half * 8;
        if (r >= nrows) continue;
        const int p = p0 + r;
        const float wrow = (EPI == MOE_UP_ACT && wgt) ? wgt[perm[p]] : 1.0f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int n = n0 + col0 + j * 8 + (lane & 3) * 2 + c;
                if (n >= N) continue;
                if (EPI == MOE_GATE_UP) {
                    const float g = acc[0][j][half * 2 + c], u = acc[NB - 1][j][half * 2 + c];
                    act[(size_t)p * N + n] = __float2bfloat16_rn(moe_glu(g, u, act_kind, limit));
                } else if (EPI == MOE_UP_ACT) {
                    act[(size_t)p * N + n] = __float2bfloat16_rn(moe_act(wrow * acc[0][j][half * 2 + c], act_kind));
                } else {
                    out2[(size_t)perm[p] * N + n] = acc[0][j][half * 2 + c];
                }
            }
        }
    }
}

// Any element type on the CUDA cores, float32 accumulation: 256 threads, a 4 x 4 patch each.
template <typename TA, int EPI>
__global__ void __launch_bounds__(256) moe_gemm_simple_kernel(const TA* __restrict__ a, const TA* __restrict__ w,
                                                              const int* __restrict__ offsets,
                                                              const int* __restrict__ tile_start,
                                                              const int* __restrict__ perm, int E, int top, int N, int K,
                                                              TA* __restrict__ act, float* __restrict__ out2,
                                                              const float* __restrict__ wgt, int act_kind, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NB = EPI == MOE_GATE_UP ? 2 : 1;
    constexpr int BK = 16;
    __shared__ float sa[BK][MOE_BM + 4];
    __shared__ float sw[NB][BK][MOE_BN + 4];
    __shared__ int src_row[MOE_BM];
    const int tile = blockIdx.x;
    if (tile >= tile_start[E]) return;
    const int e = moe_find_expert(tile_start, E, tile);
    const int p0 = offsets[e] + (tile - tile_start[e]) * MOE_BM;
    const int nrows = min(MOE_BM, offsets[e + 1] - p0);
    const int n0 = blockIdx.y * MOE_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int r = tid; r < MOE_BM; r += 256)
        src_row[r] = r < nrows ? (EPI != MOE_DOWN ? perm[p0 + r] / top : p0 + r) : -1;
    __syncthreads();
    const TA* we = w + (size_t)e * NB * N * K;
    float acc[NB][4][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[b][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int c = tid; c < MOE_BM * BK; c += 256) {
            const int r = c / BK, k = c % BK;
            const int sr = src_row[r];
            sa[k][r] = (sr >= 0 && k0 + k < K) ? to_f32(a[(size_t)sr * K + k0 + k]) : 0.f;
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
            for (int c = tid; c < MOE_BN * BK; c += 256) {
                const int r = c / BK, k = c % BK;
                sw[b][k][r] = (n0 + r < N && k0 + k < K) ? to_f32(we[((size_t)b * N + n0 + r) * K + k0 + k]) : 0.f;
            }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[4], wv[NB][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[k][ty * 4 + i];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[b][j] = sw[b][k][tx * 4 + j];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[b][i][j] = fmaf(av[i], wv[b][j], acc[b][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= nrows) continue;
        const int p = p0 + r;
        const float wrow = (EPI == MOE_UP_ACT && wgt) ? wgt[perm[p]] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (EPI == MOE_GATE_UP)
                act[(size_t)p * N + n] = from_f32<TA>(moe_glu(acc[0][i][j], acc[NB - 1][i][j], act_kind, limit));
            else if (EPI == MOE_UP_ACT)
                act[(size_t)p * N + n] = from_f32<TA>(moe_act(wrow * acc[0][i][j], act_kind));
            else
                out2[(size_t)perm[p] * N + n] = acc[0][i][j];
        }
    }
}

template <typename TA>
__global__ void moe_combine_kernel(const float* __restrict__ out2, const float* __restrict__ wgt, int top, int D,
                                   size_t total, TA* __restrict__ y, const TA* __restrict__ base, const int* __restrict__ eidx,
                                   int n_real, const TA* __restrict__ h) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / D;
        const int d = (int)(idx - t * D);
        float acc = base ? to_f32(base[idx]) : 0.f;        // wgt nullptr: a plain sum; base: added to it (a shared expert's output)
        for (int j = 0; j < top; ++j) {
            // an entry that names an expert beyond the real ones passes the layer's input on as it is
            const bool pass = eidx && eidx[t * top + j] >= n_real;
            acc += (wgt ? wgt[t * top + j] : 1.0f) * (pass ? to_f32(h[idx]) : out2[(t * top + j) * (size_t)D + d]);
        }
        y[idx] = from_f32<TA>(acc);
    }
}

// h [T, D]; wr float32 [E, D]; br float32 [E] or nullptr; idx int32 [T, top]; wgt float32 [T, top].
PICO_API int pico_moe_route(const void* h, const float* wr, const float* br, int T, int D, int E, int top, int mode,
                            int* idx, float* wgt, int dtype, const float* choice_bias, float weight_scale, int groups,
                            int groups_keep, int renorm, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E < 1 || top < 1 || top > E || top > 32 || E > 8192 || mode < 0 || mode > 2) return PICO_ERR_SIZE;
    if (groups < 1 || E % groups || groups_keep < 1 || groups_keep > groups) return PICO_ERR_SIZE;
    if ((groups > 1 || renorm) && mode != MOE_SCORE_SOFTMAX_ALL) return PICO_ERR_SIZE;
    if (renorm && !(weight_scale != 0.f)) return PICO_ERR_SIZE;
    // four tokens a block when there are many (the router matrix is read once per block), one otherwise
    const int tok = T >= 512 ? 4 : 1;
    const size_t smem = ((size_t)tok * ((D + 3) & ~3) + (size_t)3 * tok * E) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    const dim3 grid((T + tok - 1) / tok);
#define LAUNCH_ROUTE(TA, TOK)                                                                                             \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(moe_route_kernel<TA, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        pico_launch((moe_route_kernel<TA, TOK>), grid, dim3(256), smem, stream, (const TA*)h, wr, br, T, D, E, top, mode, idx, wgt, choice_bias, weight_scale, groups, groups_keep, renorm); \
    } while (0)
    if (dtype == PICO_F32) {
        if (tok == 4) LAUNCH_ROUTE(float, 4); else LAUNCH_ROUTE(float, 1);
    } else if (dtype == PICO_BF16) {
        if (tok == 4) LAUNCH_ROUTE(bf16, 4); else LAUNCH_ROUTE(bf16, 1);
    } else
        return PICO_ERR_DTYPE;
#undef LAUNCH_ROUTE
    return pico_launch_status();
}

// The most tiles of bm rows n entries over E experts can make.
static inline int moe_max_tiles(int n, int E, int bm) { return n / bm + (n < E ? n : E); }

// idx int32 [n]; offsets, tile_start int32 [E + 1]; perm int32 [n].
// Rows per tile of the grouped products for n entries over E experts: 16 while the experts' lists are short.
PICO_API int pico_moe_tile_rows(int n, int E, int dtype, int K1, int K2) {
    const bool mma = dtype == PICO_BF16 && K1 % 8 == 0 && K2 % 8 == 0;
    return mma && n <= 16 * E ? 16 : MOE_BM;
}

PICO_API int pico_moe_group(const int* idx, int n, int E, int bm, int* offsets, int* tile_start, int* perm, int* place,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (E < 1 || E > 4096 || (bm != 16 && bm != MOE_BM)) return PICO_ERR_SIZE;
    pico_launch(moe_group_kernel, dim3(1), dim3(n >= 4096 ? 1024 : 256), (size_t)2 * E * sizeof(int), stream, idx, n, E, bm,
                offsets, tile_start, perm, place);
    return pico_launch_status();
}

// The library path for many tokens: rows gathered into expert order, a library grouped product on them, and the
// weighted sum read back through ``place``.
// xs[p, :] = x[perm[p] / top, :], 16 bytes per thread and access (D * sizeof a multiple of 16).
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ perm, int top, int row16,
                                  size_t total, uint4* __restrict__ xs) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / row16;
        const int c = (int)(idx - p * row16);
        xs[idx] = x[(size_t)(perm[p] / top) * row16 + c];
    }
}

PICO_API int pico_moe_gather(const void* x, const int* perm, int n, int top, int row_bytes, void* xs, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (row_bytes % 16 != 0 || top < 1) return PICO_ERR_ALIGN;
    const size_t total = (size_t)n * (row_bytes / 16);
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    pico_launch(moe_gather_kernel, dim3(blocks), dim3(256), 0, stream, (const uint4*)x, perm, top, row_bytes / 16, total,
                (uint4*)xs);
    return pico_launch_status();
}

// y[t] = sum_j wgt[t, j] * ys[place[t * top + j]] with ys in expert order (activation type), float32 sum.
// VEC: D a multiple of 8 (bfloat16) or 4 (float32): 16 bytes per access.
template <typename TA, bool VEC>
__global__ void moe_combine_placed_kernel(const TA* __restrict__ ys, const int* __restrict__ place,
                                          const float* __restrict__ wgt, int top, int D, size_t total, TA* __restrict__ y,
                                          const TA* __restrict__ base, const int* __restrict__ eidx, int n_real,
                                          const TA* __restrict__ h) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int W = VEC ? 16 / (int)sizeof(TA) : 1;
    const int Dv = D / W;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / Dv;
        const int d = (int)(idx - t * Dv) * W;
        float acc[W];
#pragma unroll
        for (int k = 0; k < W; ++k) acc[k] = base ? to_f32(base[t * (size_t)D + d + k]) : 0.f;
        for (int j = 0; j < top; ++j) {
            const float g = wgt ? wgt[t * top + j] : 1.0f;
            const bool pass = eidx && eidx[t * top + j] >= n_real;     // an expert that hands its input on
            const TA* row = pass ? h + t * (size_t)D + d : ys + (size_t)place[t * top + j] * D + d;
            if (VEC) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row);
                const TA* v = reinterpret_cast<const TA*>(&raw);
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] += g * to_f32(v[k]);
            } else {
                acc[0] += g * to_f32(row[0]);
            }
        }
        if (VEC) {
            uint4 raw;
            TA* v = reinterpret_cast<TA*>(&raw);
#pragma unroll
            for (int k = 0; k < W; ++k) v[k] = from_f32<TA>(acc[k]);
            *reinterpret_cast<uint4*>(y + t * (size_t)D + d) = raw;
        } else {
            y[t * (size_t)D + d] = from_f32<TA>(acc[0]);
        }
    }
}

PICO_API int pico_moe_combine_placed(const void* ys, const int* place, const float* wgt, int T, int top, int D, void* y,
                                     const void* base, int dtype, const int* eidx, int n_real, const void* h,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dtype != PICO_F32 && dtype != PICO_BF16) return PICO_ERR_DTYPE;
    const int w = dtype == PICO_F32 ? 4 : 8;
    const bool vec = D % w == 0;
    const size_t total = (size_t)T * (vec ? D / w : D);
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
#define LAUNCH_CP(TA, V)                                                                                              \
    pico_launch((moe_combine_placed_kernel<TA, V>), dim3(blocks), dim3(256), 0, stream, (const TA*)ys, place, wgt, top, D, \
                total, (TA*)y, (const TA*)base, eidx, n_real, (const TA*)h)
    if (dtype == PICO_F32) {
        if (vec) LAUNCH_CP(float, true); else LAUNCH_CP(float, false);
    } else {
        if (vec) LAUNCH_CP(bf16, true); else LAUNCH_CP(bf16, false);
    }
#undef LAUNCH_CP
    return pico_launch_status();
}

// epi 0: a = x [T, K], w [E, 2N, K] -> act [n, N];  epi 1: a = act [n, K], w [E, N, K] -> out2 float32 [n, N].
// bm: the rows per tile that pico_moe_group was given (16 only for bfloat16 with K a multiple of 8).
PICO_API int pico_moe_gemm(const void* a, const void* w, const int* offsets, const int* tile_start, const int* perm,
                           int n, int E, int top, int N, int K, int epi, int bm, void* act, float* out2,
                           const float* wgt, int act_kind, float limit, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (N < 1 || K < 1 || epi < 0 || epi > 2 || act_kind < 0 || act_kind > 2 || (act_kind == MOE_ACT_CAPPED && epi != MOE_GATE_UP) || (bm != 16 && bm != MOE_BM)) return PICO_ERR_SIZE;
    if (bm == 16 && !(dtype == PICO_BF16 && K % 8 == 0)) return PICO_ERR_SIZE;
    const dim3 grid(moe_max_tiles(n, E, bm), (N + MOE_BN - 1) / MOE_BN);
    if (grid.y > 65535) return PICO_ERR_SIZE;
#define MOE_MMA(EPI_, BM_, BK_)                                                                                             \
    pico_launch((moe_gemm_mma_kernel<EPI_, BM_, BK_>), grid, dim3(128), 0, stream, (const bf16*)a, (const bf16*)w, offsets, \
                tile_start, perm, E, top, N, K, (bf16*)act, out2, wgt, act_kind, limit)
    if (dtype == PICO_BF16 && K % 8 == 0) {
        if (epi == MOE_GATE_UP) {
            if (bm == 16) MOE_MMA(MOE_GATE_UP, 16, 32); else MOE_MMA(MOE_GATE_UP, 64, 32);
        } else if (epi == MOE_UP_ACT) {
            if (bm == 16) MOE_MMA(MOE_UP_ACT, 16, 64); else MOE_MMA(MOE_UP_ACT, 64, 32);
        } else {
            if (bm == 16) MOE_MMA(MOE_DOWN, 16, 64); else MOE_MMA(MOE_DOWN, 64, 32);
        }
    } else if (dtype == PICO_BF16) {
#define MOE_SIMPLE(TA_, EPI_)                                                                                              \
    pico_launch((moe_gemm_simple_kernel<TA_, EPI_>), grid, dim3(256), 0, stream, (const TA_*)a, (const TA_*)w, offsets,     \
                tile_start, perm, E, top, N, K, (TA_*)act, out2, wgt, act_kind, limit)
        if (epi == MOE_GATE_UP) MOE_SIMPLE(bf16, MOE_GATE_UP);
        else if (epi == MOE_UP_ACT) MOE_SIMPLE(bf16, MOE_UP_ACT);
        else MOE_SIMPLE(bf16, MOE_DOWN);
    } else if (dtype == PICO_F32) {
        if (epi == MOE_GATE_UP) MOE_SIMPLE(float, MOE_GATE_UP);
        else if (epi == MOE_UP_ACT) MOE_SIMPLE(float, MOE_UP_ACT);
        else MOE_SIMPLE(float, MOE_DOWN);
#undef MOE_SIMPLE
    } else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// out2 float32 [T * top, D]; wgt float32 [T, top]; y [T, D].
PICO_API int pico_moe_combine(const float* out2, const float* wgt, int T, int top, int D, void* y, const void* base,
                              int dtype, const int* eidx, int n_real, const void* h, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t total = (size_t)T * D;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((moe_combine_kernel<float>), dim3(blocks), dim3(256), 0, stream, out2, wgt, top, D, total, (float*)y,
                    (const float*)base, eidx, n_real, (const float*)h);
    else if (dtype == PICO_BF16)
        pico_launch((moe_combine_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, out2, wgt, top, D, total, (bf16*)y,
                    (const bf16*)base, eidx, n_real, (const bf16*)h);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// out[p, :] = act(wgt[perm[p]] * u[p, :]) in float32: the activation of experts without a gate between the library's
// two grouped products (rows in expert order), with the entry's router weight acting on the expert's input.  perm and
// wgt nullptr: a plain activation over [n, ff] (a dense layer of the same form, such as a shared expert).  In place
// when out == u.
template <typename TA>
__global__ void moe_scaled_act_kernel(const TA* u, const int* __restrict__ perm, const float* __restrict__ wgt, int ff,
                                      size_t total, int act_kind, TA* out) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / ff;
        const float w = wgt ? wgt[perm ? perm[p] : p] : 1.0f;
        out[idx] = from_f32<TA>(moe_act(w * to_f32(u[idx]), act_kind));
    }
}

// bfloat16 rows of a multiple of 8 elements, 16 bytes per access.
__global__ void moe_scaled_act_bf16x8_kernel(const bf16* u, const int* __restrict__ perm, const float* __restrict__ wgt, int ff8,
                                             size_t total8, int act_kind, bf16* out) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / ff8;
        const float w = wgt ? wgt[perm ? perm[p] : p] : 1.0f;
        const uint4 raw = *reinterpret_cast<const uint4*>(u + idx * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 res;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __bfloat1622float2(h2[k]);
            o2[k] = __floats2bfloat162_rn(moe_act(w * v.x, act_kind), moe_act(w * v.y, act_kind));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = res;
    }
}

PICO_API int pico_moe_scaled_act(const void* u, const int* perm, const float* wgt, int n, int ff, int act_kind, void* out,
                                 int dtype, cudaStream_t stream) {
    if (n <= 0 || ff <= 0) return 0;
    if (act_kind < 0 || act_kind > 1) return PICO_ERR_SIZE;
    const size_t total = (size_t)n * ff;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((moe_scaled_act_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)u, perm, wgt, ff, total,
                    act_kind, (float*)out);
    else if (dtype == PICO_BF16 && ff % 8 == 0 && ((uintptr_t)u & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const size_t want8 = (total / 8 + 255) / 256;
        pico_launch(moe_scaled_act_bf16x8_kernel, dim3((int)((long long)want8 > cap ? cap : (long long)want8)), dim3(256), 0, stream,
                    (const bf16*)u, perm, wgt, ff / 8, total / 8, act_kind, (bf16*)out);
    } else if (dtype == PICO_BF16)
        pico_launch((moe_scaled_act_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)u, perm, wgt, ff, total,
                    act_kind, (bf16*)out);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
