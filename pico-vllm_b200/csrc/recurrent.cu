// Mixers whose memory is a matrix of fixed size per request, with gates that depend on the token:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T ,   o_t = S_t^T q_t         (S: [d, dv] per head, float32, kept per request)
//
// where a_t is one number per head (GATE 1) or one per head and row of S (GATE 2).  Three designs of mixer are this
// recurrence behind different gates, and each has a small kernel that turns its projections into the float32 q, k, v, a:
//
//   matrix memory with exponential gates (mlstm_*):  a = exp(f + m_(t-1) - m_t), k scaled by exp(i - m_t), with the running
//       maximum m_t = max(f + m_(t-1), i) kept per head; v gets one more column of ones, whose row of S is the normaliser n;
//   gated linear attention whose forget gate writes (hgrn2_prepare): a = f per row, k = 1 - f;
//   a state-space layer (causal_conv_silu, mamba2_prepare): a = exp(-exp(A) dt), k = B, v = dt x, q = C, after a short
//       causal convolution over x, B and C whose last inputs are part of the request's state.
//
// gated_linear_attention_kernel is the recurrence: the columns of S evolve independently of each other, so a block takes
// 64 columns of one head of one segment, a warp eight of them, a lane the rows lane, lane + 32, ... in registers; tokens
// are walked in order, eight at a time from shared memory; the state is stored transposed [slot, head, dv, d].  A segment
// of one token is a decode step; a portion of a prompt goes on from the state the portion before left.
// group_rms_norm_kernel finishes all three: optional normaliser, skip term and gate, a root mean square per group of
// columns, a weight, an optional gate, into the activation type.
//
// Everything here is float32 whatever the activation type; only the projections read and the result written are not.
#include "common.cuh"

#define GL_TOK 8
#define GL_COLS 8
#define GL_WARPS 8

__device__ __forceinline__ float rc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rc_logsigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// Chunks of a long segment (the same three passes as the constant-decay kernel of linear_attention.cu):
//   pass A (STATE_ONLY): every chunk from a zero state, no outputs, and the product of its gates per row (GATE 2) or per
//                        head (GATE 1) into chunk_gate;
//   pass B (gated_linear_scan_kernel): start state of every chunk, the request's new state;
//   pass C: every chunk again from its start state, with outputs.
__device__ __forceinline__ int gl_chunk_base(const int* __restrict__ cu_q, int seg, int chunk) {
    int base = 0;
    for (int s = 0; s < seg; ++s) base += (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
    return base;
}

// XCOL (GATE 1; dv = 64 n + 1, as when a column of ones rides with the values): the blocks cover the first dv - 1 columns
// and the first warp of the first block carries the last one as a ninth column, instead of a block for one column.
template <int DPL, int GATE, bool STATE_ONLY, bool XCOL>
__global__ void __launch_bounds__(GL_WARPS * 32)
gated_linear_attention_kernel(const float* __restrict__ q, int q_stride, const float* __restrict__ k, int k_stride,
                              const float* __restrict__ v, int v_stride, const float* __restrict__ gate, int gate_stride,
                              float* __restrict__ state, const int* __restrict__ seg_slots, const int* __restrict__ cu_q,
                              const int* __restrict__ positions, float* __restrict__ out, int out_stride, int H, int qk_rep,
                              int d, int dv, int chunk, int max_chunks, float* __restrict__ chunk_state,
                              float* __restrict__ chunk_gate) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float gsm[];
    const int dp = (d + 3) & ~3;
    float* qs = gsm;                                   // [GL_TOK][dp]
    float* ks = qs + GL_TOK * dp;                      // [GL_TOK][dp]
    float* as = ks + GL_TOK * dp;                      // [GL_TOK][dp] (GATE 2) or [GL_TOK] (GATE 1, padded to dp)
    float* vs = as + GL_TOK * dp;                      // [GL_TOK][GL_WARPS * GL_COLS]
    float* part = vs + GL_TOK * GL_WARPS * GL_COLS;    // [GL_WARPS][GL_TOK][32][GL_COLS]
    const int seg = chunk > 0 ? blockIdx.z / max_chunks : blockIdx.z, ci = chunk > 0 ? blockIdx.z % max_chunks : 0;
    const int h = blockIdx.y, col_base = blockIdx.x * (GL_WARPS * GL_COLS);
    int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (t_end <= t_begin || positions[t_begin] < 0) return;      // an empty or a padding segment
    if (chunk > 0) {
        t_begin += ci * chunk;
        if (t_begin >= t_end) return;
        t_end = min(t_end, t_begin + chunk);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = col_base + warp * GL_COLS;
    const int hq = h / qk_rep;
    const size_t cidx = chunk > 0 ? (size_t)(gl_chunk_base(cu_q, seg, chunk) + ci) * H + h : 0;
    float* st = chunk > 0 ? chunk_state + cidx * (size_t)dv * d : state + ((size_t)seg_slots[seg] * H + h) * (size_t)dv * d;
    float S[DPL][GL_COLS];
    float gprod[DPL];                                  // pass A: the product of this chunk's gates per row
#pragma unroll
    for (int r = 0; r < DPL; ++r) {
        gprod[r] = 1.0f;
#pragma unroll
        for (int c = 0; c < GL_COLS; ++c) {
            const int i = lane + 32 * r, j = col0 + c;
            S[r][c] = (!STATE_ONLY && i < d && j < dv) ? st[(size_t)j * d + i] : 0.f;
        }
    }
    float* mypart = part + (size_t)warp * GL_TOK * 32 * GL_COLS;
    const bool live = col0 < dv;                       // uniform for the warp
    const bool xcol = XCOL && blockIdx.x == 0 && warp == 0;
    const int jx = dv - 1;                             // the ninth column
    float* vxs = as + GL_TOK;                          // [GL_TOK] its values (GATE 1 leaves the room)
    float Sx[DPL];
#pragma unroll
    for (int r = 0; r < DPL; ++r) {
        const int i = lane + 32 * r;
        Sx[r] = (xcol && !STATE_ONLY && i < d) ? st[(size_t)jx * d + i] : 0.f;
    }
    // Each thread's share of eight tokens' q, k, gates and values: asked for while the eight tokens before are walked, kept
    // in registers, put into shared memory at the top of the next round.
    constexpr int NTH = GL_WARPS * 32;
    static_assert(GL_TOK * GL_WARPS * GL_COLS == 2 * NTH, "two values a thread and round");
    int pf_tt[DPL], pf_i[DPL];                         // token of the round (>= GL_TOK: none) and row of element j
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
        const int idx = threadIdx.x + j * NTH;
        pf_tt[j] = idx / d;
        pf_i[j] = idx - pf_tt[j] * d;
    }
    const int v_tt = threadIdx.x / (GL_WARPS * GL_COLS), v_c = threadIdx.x % (GL_WARPS * GL_COLS);
    const bool v_in = col_base + v_c < dv;
    float rq[DPL], rk[DPL], ra[DPL], rv[2] = {0.f, 0.f}, ra1 = 0.f, rvx = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) rq[j] = rk[j] = ra[j] = 0.f;
    auto fetch = [&](int t0, int nt) {
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            if (pf_tt[j] < nt) {
                const size_t t = (size_t)(t0 + pf_tt[j]);
                if (!STATE_ONLY) rq[j] = q[t * q_stride + hq * d + pf_i[j]];
                rk[j] = k[t * k_stride + hq * d + pf_i[j]];
                if (GATE == 2) ra[j] = gate[t * gate_stride + (size_t)h * d + pf_i[j]];
            }
        }
        if (GATE == 1 && threadIdx.x < nt) ra1 = gate[(size_t)(t0 + threadIdx.x) * gate_stride + h];
        if (XCOL && blockIdx.x == 0 && threadIdx.x >= 32 && threadIdx.x < 32 + nt)
            rvx = v[(size_t)(t0 + threadIdx.x - 32) * v_stride + (size_t)h * dv + jx];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int tt = v_tt + j * (GL_TOK / 2);
            rv[j] = (tt < nt && v_in) ? v[(size_t)(t0 + tt) * v_stride + (size_t)h * dv + col_base + v_c] : 0.f;
        }
    };
    fetch(t_begin, min(GL_TOK, t_end - t_begin));
    for (int t0 = t_begin; t0 < t_end; t0 += GL_TOK) {
        const int nt = min(GL_TOK, t_end - t0);
        __syncthreads();                               // everyone is done with the tokens before
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            if (pf_tt[j] < nt) {
                if (!STATE_ONLY) qs[pf_tt[j] * dp + pf_i[j]] = rq[j];
                ks[pf_tt[j] * dp + pf_i[j]] = rk[j];
                if (GATE == 2) as[pf_tt[j] * dp + pf_i[j]] = ra[j];
            }
        }
        if (GATE == 1 && threadIdx.x < nt) as[threadIdx.x] = ra1;
        if (XCOL && blockIdx.x == 0 && threadIdx.x >= 32 && threadIdx.x < 32 + nt) vxs[threadIdx.x - 32] = rvx;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int tt = v_tt + j * (GL_TOK / 2);
            if (tt < nt) vs[tt * (GL_WARPS * GL_COLS) + v_c] = rv[j];
        }
        __syncthreads();
        if (t0 + GL_TOK < t_end) fetch(t0 + GL_TOK, min(GL_TOK, t_end - t0 - GL_TOK));
        if (!live) continue;                           // a warp past the last column only helps to load
        for (int tt = 0; tt < nt; ++tt) {
            const float4 va = *reinterpret_cast<const float4*>(vs + tt * GL_WARPS * GL_COLS + warp * GL_COLS);
            const float4 vb = *reinterpret_cast<const float4*>(vs + tt * GL_WARPS * GL_COLS + warp * GL_COLS + 4);
            const float vv[GL_COLS] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
            float p[GL_COLS], px = 0.f;
#pragma unroll
            for (int c = 0; c < GL_COLS; ++c) p[c] = 0.f;
            const float a1 = GATE == 1 ? as[tt] : 1.0f;
#pragma unroll
            for (int r = 0; r < DPL; ++r) {
                const int i = lane + 32 * r;
                const bool in = i < d;
                const float kk = in ? ks[tt * dp + i] : 0.f;
                const float qq = (!STATE_ONLY && in) ? qs[tt * dp + i] : 0.f;
                const float a = GATE == 2 ? (in ? as[tt * dp + i] : 0.f) : a1;
                if (STATE_ONLY) gprod[r] *= a;
#pragma unroll
                for (int c = 0; c < GL_COLS; ++c) {
                    S[r][c] = fmaf(a, S[r][c], kk * vv[c]);
                    if (!STATE_ONLY) p[c] = fmaf(S[r][c], qq, p[c]);
                }
                if (XCOL && xcol) {
                    Sx[r] = fmaf(a, Sx[r], kk * vxs[tt]);
                    if (!STATE_ONLY) px = fmaf(Sx[r], qq, px);
                }
            }
            if (XCOL && xcol && !STATE_ONLY) {
                px = warp_sum(px);
                if (lane == 0) out[(size_t)(t0 + tt) * out_stride + (size_t)h * dv + jx] = px;
            }
            if (!STATE_ONLY) {
                float* dst = mypart + ((size_t)tt * 32 + lane) * GL_COLS;
                *reinterpret_cast<float4*>(dst) = make_float4(p[0], p[1], p[2], p[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(p[4], p[5], p[6], p[7]);
            }
        }
        if (!STATE_ONLY) {
            __syncwarp();
            // lane -> (tokens lane / 8 and lane / 8 + 4, column lane % 8): the sum of the 32 lanes' partials, read in a
            // rotated order so that the 32 reads of a step fall into 32 banks
            const int t4 = lane >> 3, c = lane & 7;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 8
            for (int l = 0; l < 32; ++l) {
                const int ll = (l + t4) & 31;
                if (t4 < nt) acc0 += mypart[((size_t)t4 * 32 + ll) * GL_COLS + c];
                if (t4 + 4 < nt) acc1 += mypart[((size_t)(t4 + 4) * 32 + ll) * GL_COLS + c];
            }
            const int j = col0 + c;
            if (j < dv) {
                if (t4 < nt) out[(size_t)(t0 + t4) * out_stride + (size_t)h * dv + j] = acc0;
                if (t4 + 4 < nt) out[(size_t)(t0 + t4 + 4) * out_stride + (size_t)h * dv + j] = acc1;
            }
            __syncwarp();
        }
    }
    if (STATE_ONLY || chunk == 0) {
#pragma unroll
        for (int r = 0; r < DPL; ++r)
#pragma unroll
            for (int c = 0; c < GL_COLS; ++c) {
                const int i = lane + 32 * r, j = col0 + c;
                if (i < d && j < dv) st[(size_t)j * d + i] = S[r][c];
            }
        if (XCOL && xcol) {
#pragma unroll
            for (int r = 0; r < DPL; ++r) {
                const int i = lane + 32 * r;
                if (i < d) st[(size_t)jx * d + i] = Sx[r];
            }
        }
    }
    if (STATE_ONLY && blockIdx.x == 0 && warp == 0) {
#pragma unroll
        for (int r = 0; r < DPL; ++r) {
            const int i = lane + 32 * r;
            if (i < d) chunk_gate[cidx * d + i] = gprod[r];
        }
    }
}

// Pass B: a thread per state element (column j, row i) of one (segment, head); walks the segment's chunks in order.
__global__ void __launch_bounds__(256)
gated_linear_scan_kernel(float* __restrict__ state, const int* __restrict__ seg_slots, const int* __restrict__ cu_q,
                         const int* __restrict__ positions, int H, int d, int dv, int chunk, float* __restrict__ chunk_state,
                         const float* __restrict__ chunk_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_head = d * dv;
    const int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (e >= per_head || t_end <= t_begin || positions[t_begin] < 0) return;
    const int n_chunks = (t_end - t_begin + chunk - 1) / chunk;
    const int i = e % d;
    const size_t base = (size_t)gl_chunk_base(cu_q, seg, chunk);
    float* sp = state + ((size_t)seg_slots[seg] * H + h) * (size_t)per_head + e;
    float* cs = chunk_state + (base * H + h) * (size_t)per_head + e;
    const float* cg = chunk_gate + (base * H + h) * (size_t)d + i;
    const size_t step = (size_t)H * per_head, gstep = (size_t)H * d;
    float S = *sp;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {          // the loads of eight chunks are in flight together
        float local[8], g[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            local[k] = c0 + k < n_chunks ? cs[(size_t)(c0 + k) * step] : 0.f;
            g[k] = c0 + k < n_chunks ? cg[(size_t)(c0 + k) * gstep] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (c0 + k < n_chunks) {
                cs[(size_t)(c0 + k) * step] = S;
                S = fmaf(g[k], S, local[k]);
            }
    }
    *sp = S;
}

// q, k: float32 rows (head h reads q + t * q_stride + (h / qk_rep) * d); v: float32 rows, head h at h * dv; gate float32
// rows of gate_stride with H numbers (gate_kind 1) or H * d numbers (gate_kind 2); state float32 [slots, H, dv, d]; out float32 rows of out_stride, head h at
// h * dv.  A segment whose first position is negative is padding and is skipped.  chunk > 0: the chunked form for segments
// up to max_q_len tokens; chunk_state float32 with room for (T / chunk + S) x H x dv x d, chunk_gate for (T / chunk + S) x H x d.
PICO_API int pico_gated_linear_attention(const float* q, int q_stride, const float* k, int k_stride, const float* v, int v_stride,
                                         const float* gate, int gate_stride, int gate_kind, float* state, const int* seg_slots, const int* cu_q,
                                         const int* positions, float* out, int out_stride, int S, int H, int qk_rep, int d,
                                         int dv, int chunk, int max_q_len, float* chunk_state, float* chunk_gate,
                                         cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || d < 1 || d > 256 || dv < 1 || qk_rep < 1 || H % qk_rep != 0) return PICO_ERR_SIZE;
    if (gate_kind != 1 && gate_kind != 2) return PICO_ERR_SIZE;
    if (chunk < 0 || (chunk > 0 && (!chunk_state || !chunk_gate || max_q_len < 1))) return PICO_ERR_SIZE;
    const int max_chunks = chunk > 0 ? (max_q_len + chunk - 1) / chunk : 1;
    if ((long long)S * max_chunks > 65535) return PICO_ERR_SIZE;
    const int dpl = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8;
    const int dp = (d + 3) & ~3;
    const size_t smem = ((size_t)3 * GL_TOK * dp + GL_TOK * GL_WARPS * GL_COLS + (size_t)GL_WARPS * GL_TOK * 32 * GL_COLS) * sizeof(float);
    const bool xc = gate_kind == 1 && dv > 1 && dv % (GL_WARPS * GL_COLS) == 1;      // the last column rides with a warp
    const dim3 grid(xc ? dv / (GL_WARPS * GL_COLS) : (dv + GL_WARPS * GL_COLS - 1) / (GL_WARPS * GL_COLS), H, S * max_chunks);
#define GL_LAUNCH(DPL, G, SO, XC)                                                                                        \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(gated_linear_attention_kernel<DPL, G, SO, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                             \
        pico_launch((gated_linear_attention_kernel<DPL, G, SO, XC>), grid, dim3(GL_WARPS * 32), smem, stream, q, q_stride, k, \
                    k_stride, v, v_stride, gate, gate_stride, state, seg_slots, cu_q, positions, out, out_stride, H, qk_rep, d, dv,   \
                    chunk, max_chunks, chunk_state, chunk_gate);                                                         \
    } while (0)
#define GL_BY_GATE(DPL, SO)                                                                                              \
    do {                                                                                                                 \
        if (gate_kind == 2) GL_LAUNCH(DPL, 2, SO, false);                                                                \
        else if (xc) GL_LAUNCH(DPL, 1, SO, true);                                                                        \
        else GL_LAUNCH(DPL, 1, SO, false);                                                                               \
    } while (0)
#define GL_BY_DPL(SO)                                                                                                    \
    do {                                                                                                                 \
        if (dpl == 1) GL_BY_GATE(1, SO); else if (dpl == 2) GL_BY_GATE(2, SO); else if (dpl == 4) GL_BY_GATE(4, SO);     \
        else GL_BY_GATE(8, SO);                                                                                          \
    } while (0)
    if (chunk > 0) {
        GL_BY_DPL(true);
        pico_launch(gated_linear_scan_kernel, dim3((d * dv + 255) / 256, H, S), dim3(256), 0, stream, state, seg_slots, cu_q,
                    positions, H, d, dv, chunk, chunk_state, (const float*)chunk_gate);
    }
    GL_BY_DPL(false);
#undef GL_BY_DPL
#undef GL_BY_GATE
#undef GL_LAUNCH
    return pico_launch_status();
}

// ------------------------------------------------------------------------------------------ exponential gates
// A block of one to eight warps per (head, segment): the running maximum m_t = max(f_t + m_(t-1), i_t) is a scan under the
// composition of the maps x -> max(x + a, b): inside a warp by shuffles, across the warps through shared memory, 32
// tokens a warp and round.  i = cap tanh((z_i + b_i) / cap), f = logsigmoid(cap tanh((z_f + b_f) / cap)).
// Writes, per token and head: keep = exp(f + m_(t-1) - m_t), put = exp(i - m_t), floor = exp(-m_t); m [slots, H] goes on.
#define MG_WARPS 8
template <typename TA>
__global__ void __launch_bounds__(MG_WARPS * 32)
mlstm_gates_kernel(const TA* __restrict__ proj, int row_stride, int i_off, int f_off, const float* __restrict__ i_bias,
                   const float* __restrict__ f_bias, float cap, float* __restrict__ m_state, const int* __restrict__ seg_slots,
                   const int* __restrict__ cu_q, const int* __restrict__ positions, float* __restrict__ keep,
                   float* __restrict__ put, float* __restrict__ floor_, int H) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sA[MG_WARPS], sB[MG_WARPS];
    const int h = blockIdx.x, seg = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (t_end <= t_begin || positions[t_begin] < 0) return;
    float* mp = m_state + (size_t)seg_slots[seg] * H + h;
    float m = *mp;                                    // every thread follows the block's m
    const float bi = i_bias ? i_bias[h] : 0.f, bf = f_bias ? f_bias[h] : 0.f;
    for (int t0 = t_begin; t0 < t_end; t0 += nw * 32) {
        const int t = t0 + (int)threadIdx.x;
        const bool valid = t < t_end;
        float a = 0.f, b = -INFINITY;                 // the identity map
        if (valid) {
            const float zi = to_f32(proj[(size_t)t * row_stride + i_off + h]) + bi;
            const float zf = to_f32(proj[(size_t)t * row_stride + f_off + h]) + bf;
            b = cap * tanhf(zi / cap);
            a = rc_logsigmoid(cap * tanhf(zf / cap));
        }
        float A = a, B = b;                           // the map of this warp's tokens up to and with this one
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float A0 = __shfl_up_sync(0xffffffffu, A, o), B0 = __shfl_up_sync(0xffffffffu, B, o);
            if (lane >= o) {
                B = fmaxf(B0 + A, B);
                A = A0 + A;
            }
        }
        if (lane == 31) {
            sA[warp] = A;
            sB[warp] = B;
        }
        __syncthreads();
        float m_in = m;                               // m before this warp's first token
        for (int w = 0; w < warp; ++w) m_in = fmaxf(m_in + sA[w], sB[w]);
        const float mt = fmaxf(m_in + A, B);
        float mprev = __shfl_up_sync(0xffffffffu, mt, 1);
        if (lane == 0) mprev = m_in;
        if (valid) {
            const size_t o = (size_t)t * H + h;
            keep[o] = expf(a + mprev - mt);
            put[o] = expf(b - mt);
            floor_[o] = expf(-mt);
        }
        for (int w = 0; w < nw; ++w) m = fmaxf(m + sA[w], sB[w]);            // tokens past the end are identity maps
        __syncthreads();                              // sA and sB are written again in the next round
    }
    if (threadIdx.x == 0) *mp = m;
}

// prepared row of a token: [q: H d | k: H d | v: H (dv + 1)] float32, with q * q_scale, k * put[t, h], v and a last column 1.
template <typename TA>
__global__ void mlstm_prepare_kernel(const TA* __restrict__ proj, int row_stride, int q_off, int k_off, int v_off,
                                     const float* __restrict__ put, float q_scale, int H, int d, int dv, size_t total,
                                     float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    // gridDim.y blocks per token (several when the step is short; blocks stride over the tokens): 32-bit index arithmetic
    // inside the row
    const int nqk = H * d, nv = H * (dv + 1), n = 2 * nqk + nv;
    const size_t T = total / n;
    for (size_t t = blockIdx.x; t < T; t += gridDim.x) {
        const TA* row = proj + t * row_stride;
        float* o = out + t * n;
        const int c0 = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
        for (int c = c0; c < nqk; c += step) {
            o[c] = to_f32(row[q_off + c]) * q_scale;
            o[nqk + c] = to_f32(row[k_off + c]) * put[t * H + c / d];
        }
        for (int c = c0; c < nv; c += step) {
            const int hv = c / (dv + 1), j = c - hv * (dv + 1);
            o[2 * nqk + c] = j < dv ? to_f32(row[v_off + hv * dv + j]) : 1.0f;
        }
    }
}

PICO_API int pico_mlstm_prepare(const void* proj, int row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                                const float* i_bias, const float* f_bias, float cap, float q_scale, float* m_state,
                                const int* seg_slots, const int* cu_q, const int* positions, float* keep, float* put,
                                float* floor_, float* prepared, int T, int S, int H, int d, int dv, int dtype,
                                cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || d < 1 || dv < 1 || !(cap > 0.f)) return PICO_ERR_SIZE;
    const size_t total = (size_t)T * ((size_t)2 * H * d + (size_t)H * (dv + 1));
    const long long capb = 16LL * pico_num_sms();
    const int blocks = (int)((long long)T > capb ? capb : (long long)T);
    const int per_seg = (T + S - 1) / S;              // single tokens: a warp; long portions: eight
    const int gate_threads = per_seg <= 32 ? 32 : per_seg <= 128 ? 128 : MG_WARPS * 32;
#define ML_LAUNCH(TA)                                                                                                   \
    do {                                                                                                                \
        pico_launch((mlstm_gates_kernel<TA>), dim3(H, S), dim3(gate_threads), 0, stream, (const TA*)proj, row_stride, i_off, f_off, \
                    i_bias, f_bias, cap, m_state, seg_slots, cu_q, positions, keep, put, floor_, H);                    \
        pico_launch((mlstm_prepare_kernel<TA>), dim3(blocks, T < 512 ? 8 : 1), dim3(256), 0, stream, (const TA*)proj, row_stride, q_off, k_off, \
                    v_off, (const float*)put, q_scale, H, d, dv, total, prepared);                                      \
    } while (0)
    if (dtype == PICO_F32) ML_LAUNCH(float);
    else if (dtype == PICO_BF16) ML_LAUNCH(bf16);
    else return PICO_ERR_DTYPE;
#undef ML_LAUNCH
    return pico_launch_status();
}

// ------------------------------------------------------------------------------------------ a forget gate that writes
// prepared row of a token: [q: H d | k: H d | f: H d | v: H dv] float32 with q = silu(z_q), f = low + (1 - low) sigmoid(z_f + b),
// k = 1 - f.
template <typename TA>
__global__ void hgrn2_prepare_kernel(const TA* __restrict__ proj, int row_stride, int q_off, int f_off, int v_off,
                                     const float* __restrict__ f_bias, const float* __restrict__ lower, int nqk, int nv,
                                     size_t total, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = 3 * nqk + nv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int c = (int)(idx - t * n);
        const TA* row = proj + t * row_stride;
        float val;
        if (c < nqk) val = rc_silu(to_f32(row[q_off + c]));
        else if (c < 3 * nqk) {
            const int e = (c - nqk) % nqk;
            const float lo = lower ? lower[e] : 0.f;
            const float f = lo + (1.0f - lo) * rc_sigmoid(to_f32(row[f_off + e]) + (f_bias ? f_bias[e] : 0.f));
            val = c < 2 * nqk ? 1.0f - f : f;
        } else val = to_f32(row[v_off + c - 3 * nqk]);
        out[idx] = val;
    }
}

PICO_API int pico_hgrn2_prepare(const void* proj, int row_stride, int q_off, int f_off, int v_off, const float* f_bias,
                                const float* lower, float* prepared, int T, int nqk, int nv, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (nqk < 1 || nv < 1) return PICO_ERR_SIZE;
    const size_t total = (size_t)T * ((size_t)3 * nqk + nv);
    const long long capb = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > capb ? capb : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((hgrn2_prepare_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)proj, row_stride, q_off, f_off,
                    v_off, f_bias, lower, nqk, nv, total, prepared);
    else if (dtype == PICO_BF16)
        pico_launch((hgrn2_prepare_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)proj, row_stride, q_off, f_off,
                    v_off, f_bias, lower, nqk, nv, total, prepared);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// ------------------------------------------------------------------------------------------ a short causal convolution
// out[t, c] = silu( b[c] + sum_j w[c, j] * in(t - (taps - 1) + j, c) ), the last tap the token's own input.  Inputs before
// the segment's first token come from the request's state [slots, taps - 1, C] (its last taps - 1 inputs, oldest first; zero
// at a request's start).  conv_state_kernel, launched after, leaves the segment's last taps - 1 inputs there.
#define CONV_MAX_TAPS 16
#define CV_TOK 8
template <typename TA, int M>      // M: the taps the registers hold (4 or CONV_MAX_TAPS)
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const TA* __restrict__ proj, int row_stride, int c_off, const float* __restrict__ w,
                        const float* __restrict__ b, const float* __restrict__ conv_state, const int* __restrict__ tok_seg,
                        const int* __restrict__ seg_slots, const int* __restrict__ cu_q, const int* __restrict__ positions,
                        int C, int taps, int T, int tpb, float* __restrict__ out, int act) {
    pdl_launch_dependents();
    pdl_wait();
    // a block takes tpb consecutive tokens (one when the step is short) of 256 channels, a thread one channel: it walks the
    // tokens with the last inputs of its channel in registers (the newest at the right end, the weights likewise), so every input is read once
    const int tb = blockIdx.x * tpb, te = min(T, tb + tpb);
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < C) {
        float wt[M], win[M];
#pragma unroll
        for (int k = 0; k < M; ++k) {
            wt[M - 1 - k] = k < taps ? w[(size_t)c * taps + taps - 1 - k] : 0.f;
            win[k] = 0.f;
        }
        const float bias = b ? b[c] : 0.f;
        bool have = false;
        for (int t = tb; t < te; ++t) {
            if (positions[t] < 0) {
                out[(size_t)t * C + c] = 0.f;
                have = false;
                continue;
            }
            const int seg = tok_seg[t], begin = cu_q[seg];
            if (!have || t == begin) {                 // the inputs before this token: of this step, or kept by the request
                const float* st = conv_state + (size_t)seg_slots[seg] * (taps - 1) * C;
#pragma unroll
                for (int k = 1; k < M; ++k) {
                    if (k < taps) {
                        const int src = t - k;
                        win[M - 1 - k] = src >= begin ? to_f32(proj[(size_t)src * row_stride + c_off + c])
                                                      : st[(size_t)(taps - 1 + src - begin) * C + c];
                    }
                }
                have = true;
            }
            win[M - 1] = to_f32(proj[(size_t)t * row_stride + c_off + c]);
            float acc = bias;
#pragma unroll
            for (int k = 0; k < M; ++k) acc = fmaf(wt[k], win[k], acc);      // oldest first; unused taps weigh zero
            out[(size_t)t * C + c] = act ? rc_silu(acc) : acc;
#pragma unroll
            for (int k = 0; k < M - 1; ++k) win[k] = win[k + 1];
        }
    }
}

template <typename TA>
__global__ void conv_state_kernel(const TA* __restrict__ proj, int row_stride, int c_off, float* __restrict__ conv_state,
                                  const int* __restrict__ seg_slots, const int* __restrict__ cu_q,
                                  const int* __restrict__ positions, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    const int begin = cu_q[seg], end = cu_q[seg + 1];
    if (c >= C || end <= begin || positions[begin] < 0) return;
    float* st = conv_state + (size_t)seg_slots[seg] * (taps - 1) * C;
    float keep[CONV_MAX_TAPS];
    const int n = end - begin;
    for (int i = 0; i < taps - 1; ++i) {
        const int src = end - (taps - 1) + i;
        keep[i] = src >= begin ? to_f32(proj[(size_t)src * row_stride + c_off + c]) : st[(size_t)(i + n) * C + c];
    }
    for (int i = 0; i < taps - 1; ++i) st[(size_t)i * C + c] = keep[i];
}

// proj rows in the activation type, the C convolved channels at c_off; w float32 [C, taps]; b float32 [C] or nullptr;
// conv_state float32 [slots, taps - 1, C]; out float32 [T, C].
PICO_API int pico_causal_conv_silu(const void* proj, int row_stride, int c_off, const float* w, const float* b,
                                   float* conv_state, const int* tok_seg, const int* seg_slots, const int* cu_q,
                                   const int* positions, float* out, int T, int S, int C, int taps, int dtype, int act,
                                   cudaStream_t stream) {
    if (T <= 0 || S <= 0) return 0;
    if (C < 1 || taps < 1 || taps > CONV_MAX_TAPS || S > 65535 || (C + 255) / 256 > 65535) return PICO_ERR_SIZE;
    const int tpb = T >= 32 * CV_TOK ? CV_TOK : 1;
    const int blocks = (T + tpb - 1) / tpb;
#define CV_LAUNCH(TA)                                                                                                    \
    do {                                                                                                                 \
        if (taps <= 4)                                                                                                   \
            pico_launch((causal_conv_silu_kernel<TA, 4>), dim3(blocks, (C + 255) / 256), dim3(256), 0, stream, (const TA*)proj,  \
                        row_stride, c_off, w, b, (const float*)conv_state, tok_seg, seg_slots, cu_q, positions, C, taps, T, tpb, out, act); \
        else                                                                                                             \
            pico_launch((causal_conv_silu_kernel<TA, CONV_MAX_TAPS>), dim3(blocks, (C + 255) / 256), dim3(256), 0, stream, (const TA*)proj, \
                        row_stride, c_off, w, b, (const float*)conv_state, tok_seg, seg_slots, cu_q, positions, C, taps, T, tpb, out, act); \
        if (taps > 1)                                                                                                    \
            pico_launch((conv_state_kernel<TA>), dim3((C + 127) / 128, S), dim3(128), 0, stream, (const TA*)proj, row_stride, \
                        c_off, conv_state, seg_slots, cu_q, positions, C, taps);                                         \
    } while (0)
    if (dtype == PICO_F32) CV_LAUNCH(float);
    else if (dtype == PICO_BF16) CV_LAUNCH(bf16);
    else return PICO_ERR_DTYPE;
#undef CV_LAUNCH
    return pico_launch_status();
}

// Step size and decay of a state-space layer: dt = softplus(z_dt + dt_bias[h]); keep[t, h] = exp(-exp(A_log[h]) dt);
// vdt[t, h, :] = dt * x[t, h, :] (x float32 rows of x_stride, head h at h * dv).
template <typename TA>
__global__ void mamba2_prepare_kernel(const TA* __restrict__ proj, int row_stride, int dt_off, const float* __restrict__ dt_bias,
                                      const float* __restrict__ a_log, const float* __restrict__ x, int x_stride, int H, int dv,
                                      int T, float* __restrict__ keep, float* __restrict__ vdt) {
    pdl_launch_dependents();
    pdl_wait();
    // gridDim.y blocks per token (several when the step is short; blocks stride over the tokens): the step sizes of the
    // token's heads once into shared memory, then the products
    extern __shared__ float dts[];                     // [H]
    const int n = H * dv;
    for (size_t t = blockIdx.x; t < (size_t)T; t += gridDim.x) {
        __syncthreads();                               // the token before is done with dts
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float dt = rc_softplus(to_f32(proj[t * row_stride + dt_off + h]) + (dt_bias ? dt_bias[h] : 0.f));
            dts[h] = dt;
            if (blockIdx.y == 0) keep[t * H + h] = expf(-expf(a_log[h]) * dt);
        }
        __syncthreads();
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x)
            vdt[t * n + c] = dts[c / dv] * x[t * x_stride + c];
    }
}

PICO_API int pico_mamba2_prepare(const void* proj, int row_stride, int dt_off, const float* dt_bias, const float* a_log,
                                 const float* x, int x_stride, float* keep, float* vdt, int T, int H, int dv, int dtype,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H < 1 || H > 8192 || dv < 1) return PICO_ERR_SIZE;
    const long long capb = 16LL * pico_num_sms();
    const dim3 grid((int)((long long)T > capb ? capb : (long long)T), T < 512 ? 4 : 1);
    const size_t smem = (size_t)H * sizeof(float);
    if (dtype == PICO_F32)
        pico_launch((mamba2_prepare_kernel<float>), grid, dim3(256), smem, stream, (const float*)proj, row_stride, dt_off,
                    dt_bias, a_log, x, x_stride, H, dv, T, keep, vdt);
    else if (dtype == PICO_BF16)
        pico_launch((mamba2_prepare_kernel<bf16>), grid, dim3(256), smem, stream, (const bf16*)proj, row_stride, dt_off,
                    dt_bias, a_log, x, x_stride, H, dv, T, keep, vdt);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// ------------------------------------------------------------------------------------------ the norm that finishes them
// A warp per (token, group), four groups a block - or, for groups of 512 columns and more (WIDE), a block per (token,
// group).  For column j of group g (col = g * n + j):
//   val = x[t, g * group_stride + j]
//   den_floor:  val /= max(|x[t, g * group_stride + n]|, den_floor[t, g]) + 1e-6      (the normaliser rides as column n)
//   skip:       val += skip_w[col / skip_head] * skip[t, col]
//   pre_gate:   val *= silu(pre_gate[t, col])
//   y[t, col] = val / sqrt(mean_j val^2 + eps) * w[col] * sigmoid(post_gate[t, col])       (w, post_gate optional)
template <typename TA, bool WIDE>
__global__ void __launch_bounds__(256)
group_rms_norm_kernel(const float* __restrict__ x, int x_stride, int group_stride, int groups, int n, const float* __restrict__ w,
                      float eps, const float* __restrict__ den_floor, const float* __restrict__ skip, int skip_stride,
                      const float* __restrict__ skip_w, int skip_head, const TA* __restrict__ pre_gate, int pre_stride,
                      const TA* __restrict__ post_gate, int post_stride, TA* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const int g = WIDE ? blockIdx.y : blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int tid = WIDE ? threadIdx.x : threadIdx.x & 31, nth = WIDE ? blockDim.x : 32;
    if (g >= groups) return;                           // whole warps only, and none in the WIDE form
    {
        const float* xg = x + t * x_stride + (size_t)g * group_stride;
        float inv_den = 1.0f;
        if (den_floor) inv_den = 1.0f / (fmaxf(fabsf(xg[n]), den_floor[t * groups + g]) + 1e-6f);
        auto value = [&](int j) {
            const int col = g * n + j;
            float val = xg[j];
            if (den_floor) val *= inv_den;
            if (skip) val = fmaf(skip_w[col / skip_head], skip[t * skip_stride + col], val);
            if (pre_gate) val *= rc_silu(to_f32(pre_gate[t * pre_stride + col]));
            return val;
        };
        float ss = 0.f;
        for (int j = tid; j < n; j += nth) {
            const float val = value(j);
            ss += val * val;
        }
        const float inv = 1.0f / sqrtf((WIDE ? block_sum(ss, scratch) : warp_sum(ss)) / (float)n + eps);
        for (int j = tid; j < n; j += nth) {
            const int col = g * n + j;
            float o = value(j) * inv * (w ? w[col] : 1.0f);
            if (post_gate) o *= rc_sigmoid(to_f32(post_gate[t * post_stride + col]));
            y[t * ((size_t)groups * n) + col] = from_f32<TA>(o);
        }
    }
}

PICO_API int pico_group_rms_norm(const float* x, int x_stride, int group_stride, int groups, int n, const float* w, float eps,
                                 const float* den_floor, const float* skip, int skip_stride, const float* skip_w, int skip_head,
                                 const void* pre_gate, int pre_stride, const void* post_gate, int post_stride, void* y, int T,
                                 int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (groups < 1 || n < 1 || (skip && (!skip_w || skip_head < 1))) return PICO_ERR_SIZE;
    if (groups > 65535 * 4) return PICO_ERR_SIZE;
    const bool wide = n >= 512;
    const dim3 grid(T, wide ? groups : (groups + 3) / 4), block(wide ? 256 : 128);
#define GN_LAUNCH(TA, W)                                                                                                 \
    pico_launch((group_rms_norm_kernel<TA, W>), grid, block, 0, stream, x, x_stride, group_stride, groups, n, w, eps,     \
                den_floor, skip, skip_stride, skip_w, skip_head, (const TA*)pre_gate, pre_stride, (const TA*)post_gate,  \
                post_stride, (TA*)y)
    if (dtype == PICO_F32) { if (wide) GN_LAUNCH(float, true); else GN_LAUNCH(float, false); }
    else if (dtype == PICO_BF16) { if (wide) GN_LAUNCH(bf16, true); else GN_LAUNCH(bf16, false); }
    else
        return PICO_ERR_DTYPE;
#undef GN_LAUNCH
    return pico_launch_status();
}
