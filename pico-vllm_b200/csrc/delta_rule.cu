// The gated delta rule: a matrix memory per head and request whose rows decay and whose write is corrected by what the
// memory already holds under the key,
//
//   S <- diag(a_t) S ;   u = beta_t (v_t - S^T k_t) ;   S <- S + k_t u^T ;   o_t = S^T q_t          (S: [d, dv], float32)
//
// token by token, the read seeing the write.  With the decayed memory S' = diag(a_t) S both sums over rows are taken in one
// pass,  r1 = S'^T k_t  and  r2 = S'^T q_t :  u = beta_t (v_t - r1),  o_t = r2 + u (k_t . q_t),  so a token costs one pass
// over the registers, one reduction and one update.
//
// delta_prepare_kernel makes the float32 inputs of the recurrence from the projections: q and k as unit vectors per head
// (q times d^-1/2), beta = sigmoid, the decay a = exp(-exp(A_log) softplus(z + bias)) per head and row, and k . q.
// gated_delta_rule_kernel is the recurrence: the columns of S evolve independently of each other, so a block takes
// 16 columns of one head of one segment, eight or sixteen lanes a column with the rows dealt out among them in
// registers; the state is stored transposed [slot, head, dv, d].  A token's q, k and decay pass through shared
// memory, DR_TOK tokens at a time, the next ones' loads in flight (cp.async) while these are walked.  A segment of one token is a decode step; a
// portion of a prompt goes on from the state the portion before left.
//
// Everything here is float32 whatever the activation type; only the projections read are not.
#include "common.cuh"

#define DR_TOK 8

__device__ __forceinline__ float dr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// Grid (tokens, 1 + H): block y = 0 makes the unit vectors and k . q of all query/key heads (a warp a head), block y = h + 1
// the decays and beta of head h.  xc float32 [T, >= q_off.. ] holds the convolved q and k (G heads of d each); proj
// (activation type) holds one beta logit per head at b_off; dt [T, H * d] (activation type) the decay's argument before
// its bias.  prep float32 [T, P] with P = 2 G d + H d + H + G:  q | k | a | beta | k . q.
template <typename TA>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ xc, int xc_stride, int q_off, int k_off, const TA* __restrict__ proj,
                     int proj_stride, int b_off, const TA* __restrict__ dt, int dt_stride, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, float* __restrict__ prep, int P, int H, int G, int d, float q_scale,
                     float unit_eps) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* out = prep + t * P;
    if (blockIdx.y > 0) {
        const int h = blockIdx.y - 1;
        const float rate = expf(a_log[h]);
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float z = to_f32(dt[t * dt_stride + h * d + i]) + (dt_bias ? dt_bias[h * d + i] : 0.f);
            out[2 * G * d + h * d + i] = expf(-rate * dr_softplus(z));
        }
        if (threadIdx.x == 0) out[2 * G * d + H * d + h] = dr_sigmoid(to_f32(proj[t * proj_stride + b_off + h]));
        return;
    }
    const float* row = xc + t * xc_stride;
    for (int g = warp; g < G; g += nw) {
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float a = row[q_off + g * d + i], b = row[k_off + g * d + i];
            sq += a * a;
            sk += b * b;
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float iq = q_scale / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
        float kq = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float a = row[q_off + g * d + i] * iq, b = row[k_off + g * d + i] * ik;
            out[g * d + i] = a;
            out[G * d + g * d + i] = b;
            kq += a * b;
        }
        kq = warp_sum(kq);
        if (lane == 0) out[2 * G * d + H * d + H + g] = kq;
    }
}

PICO_API int pico_delta_prepare(const float* xc, int xc_stride, int q_off, int k_off, const void* proj, int proj_stride,
                                int b_off, const void* dt, int dt_stride, const float* dt_bias, const float* a_log,
                                float* prep, int T, int H, int G, int d, float q_scale, float unit_eps, int dtype,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H < 1 || G < 1 || H % G || d < 1 || H + 1 > 65535) return PICO_ERR_SIZE;
    const int P = 2 * G * d + H * d + H + G;
    const dim3 grid(T, 1 + H);
    if (dtype == PICO_F32)
        pico_launch((delta_prepare_kernel<float>), grid, dim3(128), 0, stream, xc, xc_stride, q_off, k_off,
                    (const float*)proj, proj_stride, b_off, (const float*)dt, dt_stride, dt_bias, a_log, prep, P, H, G, d,
                    q_scale, unit_eps);
    else if (dtype == PICO_BF16)
        pico_launch((delta_prepare_kernel<bf16>), grid, dim3(128), 0, stream, xc, xc_stride, q_off, k_off,
                    (const bf16*)proj, proj_stride, b_off, (const bf16*)dt, dt_stride, dt_bias, a_log, prep, P, H, G, d,
                    q_scale, unit_eps);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void dr_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// prep: the rows delta_prepare_kernel wrote (q at 0, k at G d, a at 2 G d, beta and k . q after them); v float32 rows with
// head h's values at h * dv; state float32 [slots, H, dv, d]; out float32 [T, H * dv].  Grid (column tiles, H, segments).
// A column is held by LPC lanes of a warp; lane l of a column holds the rows 4 l .. 4 l + 3, 4 LPC + 4 l .., ... (RPL of
// them), so a sum over rows is RPL multiply-adds in a lane (four chains side by side) and log2(LPC) exchanges among the lanes: the
// token-to-token chain - decay, two sums, write - is what sets this kernel's time, since tokens cannot run side by side.
template <int RPL, int LPC>      // rows a lane, lanes a column (8 or 16): a block holds 16 columns in 16 * LPC threads
__global__ void __launch_bounds__(16 * LPC)
gated_delta_rule_kernel(const float* __restrict__ prep, int P, const float* __restrict__ v, int v_stride,
                        float* __restrict__ state, const int* __restrict__ seg_slots, const int* __restrict__ cu_q,
                        const int* __restrict__ positions, float* __restrict__ out, int out_stride, int H, int G, int d,
                        int dv) {
    // The kernel that follows is released at the end, not here: its blocks, resident and waiting beside this kernel's
    // few warps, made the token loop 2.7 times slower (2.0 instead of 0.76 ms for 2,048 tokens).
    pdl_wait();
    extern __shared__ __align__(16) float dsm[];
    constexpr int dp = RPL * LPC;
    constexpr int NC = 16, CPW = 32 / LPC, NTH = 16 * LPC;
    // two buffers of DR_TOK tokens: q [dp], k [dp], a [dp], v [NC], beta, kq, and two floats that keep a token 16-byte aligned
    constexpr int tok_floats = 3 * dp + NC + 4;
    const int seg = blockIdx.z, h = blockIdx.y, col_base = blockIdx.x * NC;
    const int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (t_end <= t_begin || positions[t_begin] < 0) return;      // an empty or a padding segment
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPC, cw = lane / LPC;                  // row lane and column of the warp
    const int col = col_base + warp * CPW + cw;
    const int hq = h / (H / G);
    float* st = state + ((size_t)seg_slots[seg] * H + h) * (size_t)dv * d;
    float S[RPL];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = 4 * sub + 4 * LPC * (r >> 2) + (r & 3);  // four neighbouring rows at a time: one 16-byte load a token
        S[r] = (i < d && col < dv) ? st[(size_t)col * d + i] : 0.f;
    }
    const int q_at = hq * d, k_at = G * d + hq * d, a_at = 2 * G * d + h * d, b_at = 2 * G * d + H * d + h,
              kq_at = 2 * G * d + H * d + H + hq;
    auto fetch = [&](int t0, int nt, float* buf) {
        for (int idx = threadIdx.x; idx < nt * dp; idx += NTH) {
            const int tt = idx / dp, i = idx - tt * dp;
            float* dst = buf + tt * tok_floats;
            if (i < d) {
                const float* src = prep + (size_t)(t0 + tt) * P;
                dr_cp4(dst + i, src + q_at + i);
                dr_cp4(dst + dp + i, src + k_at + i);
                dr_cp4(dst + 2 * dp + i, src + a_at + i);
            } else {
                dst[i] = 0.f;
                dst[dp + i] = 0.f;
                dst[2 * dp + i] = 1.f;
            }
        }
        for (int idx = threadIdx.x; idx < nt * (NC + 2); idx += NTH) {
            const int tt = idx / (NC + 2), c = idx - tt * (NC + 2);
            float* dst = buf + tt * tok_floats + 3 * dp;
            const float* src = prep + (size_t)(t0 + tt) * P;
            if (c < NC) {
                if (col_base + c < dv) dr_cp4(dst + c, v + (size_t)(t0 + tt) * v_stride + (size_t)h * dv + col_base + c);
                else dst[c] = 0.f;
            } else if (c == NC) dr_cp4(dst + c, src + b_at);
            else dr_cp4(dst + c, src + kq_at);
        }
        dr_commit();
    };
    float* buf0 = dsm;
    float* buf1 = dsm + DR_TOK * tok_floats;
    fetch(t_begin, min(DR_TOK, t_end - t_begin), buf0);
    int turn = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += DR_TOK, turn ^= 1) {
        const int nt = min(DR_TOK, t_end - t0);
        dr_wait_all();
        __syncthreads();                    // these tokens are in; everyone is done with the other buffer
        if (t0 + DR_TOK < t_end) fetch(t0 + DR_TOK, min(DR_TOK, t_end - t0 - DR_TOK), turn ? buf0 : buf1);
        const float* buf = turn ? buf1 : buf0;
        float4 nq[RPL / 4], nk[RPL / 4], na[RPL / 4];      // the next token's rows, asked for a token ahead
        auto rows_of = [&](int tt) {
            const float* tk = buf + tt * tok_floats + 4 * sub;
#pragma unroll
            for (int j = 0; j < RPL / 4; ++j) {
                nq[j] = *reinterpret_cast<const float4*>(tk + 4 * LPC * j);
                nk[j] = *reinterpret_cast<const float4*>(tk + dp + 4 * LPC * j);
                na[j] = *reinterpret_cast<const float4*>(tk + 2 * dp + 4 * LPC * j);
            }
        };
        rows_of(0);
        for (int tt = 0; tt < nt; ++tt) {
            const float* tk = buf + tt * tok_floats;
            float p1[4] = {0.f, 0.f, 0.f, 0.f}, p2[4] = {0.f, 0.f, 0.f, 0.f};
            float kr[RPL];
#pragma unroll
            for (int j = 0; j < RPL / 4; ++j) {
                const float qv[4] = {nq[j].x, nq[j].y, nq[j].z, nq[j].w}, kv[4] = {nk[j].x, nk[j].y, nk[j].z, nk[j].w},
                            av[4] = {na[j].x, na[j].y, na[j].z, na[j].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = 4 * j + e;
                    const float s = S[r] * av[e];
                    kr[r] = kv[e];
                    S[r] = s;
                    p1[e] = fmaf(s, kv[e], p1[e]);
                    p2[e] = fmaf(s, qv[e], p2[e]);
                }
            }
            if (tt + 1 < nt) rows_of(tt + 1);
            float r1 = (p1[0] + p1[1]) + (p1[2] + p1[3]), r2 = (p2[0] + p2[1]) + (p2[2] + p2[3]);
#pragma unroll
            for (int o = LPC / 2; o > 0; o >>= 1) {
                r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                r2 += __shfl_xor_sync(0xffffffffu, r2, o);
            }
            const float u = tk[3 * dp + NC] * (tk[3 * dp + warp * CPW + cw] - r1);
#pragma unroll
            for (int r = 0; r < RPL; ++r) S[r] = fmaf(kr[r], u, S[r]);
            if (sub == 0 && col < dv)
                out[(size_t)(t0 + tt) * out_stride + (size_t)h * dv + col] = fmaf(u, tk[3 * dp + NC + 1], r2);
        }
    }
    pdl_launch_dependents();
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = 4 * sub + 4 * LPC * (r >> 2) + (r & 3);
        if (i < d && col < dv) st[(size_t)col * d + i] = S[r];
    }
}

PICO_API int pico_gated_delta_rule(const float* prep, const float* v, int v_stride, float* state, const int* seg_slots,
                                   const int* cu_q, const int* positions, float* out, int out_stride, int S, int H, int G,
                                   int d, int dv, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H < 1 || G < 1 || H % G || d < 1 || d > 256 || dv < 1) return PICO_ERR_SIZE;
    const int P = 2 * G * d + H * d + H + G;
    const dim3 grid((dv + 15) / 16, H, S);
    if (grid.z > 65535 || grid.y > 65535) return PICO_ERR_SIZE;
    // A grid that fits on the device one block to a multiprocessor asks for more shared memory than half of one, so that
    // no two blocks share a multiprocessor: released early behind a kernel that is still draining, the blocks of a
    // 2,048-token prompt landed four to a multiprocessor on the first ones that had room and took 1.5 ms instead of 0.8.
    const bool alone = (long long)grid.x * grid.y * grid.z <= pico_num_sms();
#define DR_LAUNCH(N, L)                                                                                                     \
    do {                                                                                                                    \
        size_t smem = (size_t)2 * DR_TOK * (3 * N * L + 16 + 4) * sizeof(float);                                            \
        if (alone && smem < 116 * 1024) smem = 116 * 1024;                                                                  \
        if (smem > 48 * 1024)                                                                                               \
            cudaFuncSetAttribute(gated_delta_rule_kernel<N, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        pico_launch((gated_delta_rule_kernel<N, L>), grid, dim3(16 * L), smem, stream, prep, P, v, v_stride, state,         \
                    seg_slots, cu_q, positions, out, out_stride, H, G, d, dv);                                              \
    } while (0)
    // keys of up to 32: eight lanes a column (four warps a block); longer keys: sixteen (eight warps), so that a
    // multiprocessor's four schedulers each have two warps to choose from
    if (d <= 32) DR_LAUNCH(4, 8);
    else if (d <= 64) DR_LAUNCH(4, 16);
    else if (d <= 128) DR_LAUNCH(8, 16);
    else DR_LAUNCH(16, 16);
#undef DR_LAUNCH
    return pico_launch_status();
}
