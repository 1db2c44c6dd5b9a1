// Several sublayer outputs added to the residual stream at once, each on its way through a norm of its own or none, and the
// stream handed on to whoever reads next:
//
//   x <- x + sum_i s_i * N_i(d_i)          N_i(u) = u / sqrt(mean(u^2) + eps_i) * w_i   or  u itself   (up to three terms)
//   y  = N(x)  (RMS with a weight),  or x itself in the activation type (COPY),  or nothing
//
// for layers whose mixer and feed-forward read the same normed input and whose outputs meet in one add, and for mixers
// whose two sides are normed before they are averaged.  A block per row, the row in shared memory; float32 throughout.
//
// Also here, for what a layer takes from the token itself and for feed-forward activations with a cap:
//   gelu_gate_rows_kernel   g[t, :] = gelu_tanh(z[t, :]) * table[token[t], off : off + n]
//   capped_glu_kernel       y = g' sigmoid(alpha g') (u' + 1),  g' = min(g, limit),  u' = clamp(u, -limit, limit),  optionally
//                           times sigmoid of one more number of the row
#include "common.cuh"

enum { SAN_NONE = 0, SAN_RMS = 1, SAN_COPY = 3 };

struct SumTerm {
    const void* delta;      // [*, H] in the activation type, or nullptr: no such term
    const float* w;         // weight of its norm (nullptr: none)
    int kind;               // SAN_NONE or SAN_RMS
    float eps;
    float scale;
};

template <typename TA>
__global__ void sum_add_norm_kernel(float* __restrict__ x, SumTerm t0, SumTerm t1, SumTerm t2, const float* __restrict__ w,
                                    int kind, float eps, TA* __restrict__ out, const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];      // the stream's row and the three terms' rows [4][H], 33 of scratch
    float* acc = sm;
    float* scratch = sm + 4 * (size_t)H;
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const SumTerm terms[3] = {t0, t1, t2};
    // every load of the row - the stream and all terms - is issued before anything is waited for
    float ss[3] = {0.f, 0.f, 0.f};
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        acc[i] = x[src + i];
#pragma unroll
        for (int k = 0; k < 3; ++k)
            if (terms[k].delta) {
                const float v = to_f32(((const TA*)terms[k].delta)[src + i]);
                acc[(k + 1) * (size_t)H + i] = v;
                ss[k] = fmaf(v, v, ss[k]);
            }
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const SumTerm tm = terms[k];
        if (!tm.delta) continue;
        float inv = tm.scale;
        if (tm.kind == SAN_RMS) inv *= 1.0f / sqrtf(block_sum(ss[k], scratch) / (float)H + tm.eps);
        const float* cur = acc + (k + 1) * (size_t)H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) acc[i] += cur[i] * inv * (tm.kind == SAN_RMS && tm.w ? tm.w[i] : 1.0f);
    }
    if (!rows)
        for (int i = threadIdx.x; i < H; i += blockDim.x) x[src + i] = acc[i];
    if (!out || kind == SAN_NONE) return;
    float inv = 1.0f;
    if (kind == SAN_RMS) {
        float s2 = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) s2 = fmaf(acc[i], acc[i], s2);
        inv = 1.0f / sqrtf(block_sum(s2, scratch) / (float)H + eps);
    }
    TA* dst = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TA>(kind == SAN_RMS ? acc[i] * inv * (w ? w[i] : 1.0f) : acc[i]);
}

// x float32 [*, H]; d0..d2 [*, H] in the activation type or nullptr (kinds SAN_NONE / SAN_RMS); out [R, H] or nullptr;
// rows int32 [R] or nullptr (then x is left alone).
PICO_API int pico_sum_add_norm(float* x, const void* d0, const float* w0, int k0, float e0, float s0, const void* d1,
                               const float* w1, int k1, float e1, float s1, const void* d2, const float* w2, int k2, float e2,
                               float s2, const float* w, int kind, float eps, void* out, const int* rows, int R, int H,
                               int act_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    for (int k : {k0, k1, k2})
        if (k != SAN_NONE && k != SAN_RMS) return PICO_ERR_SIZE;
    if (kind != SAN_NONE && kind != SAN_RMS && kind != SAN_COPY) return PICO_ERR_SIZE;
    const size_t smem = (size_t)(4 * (size_t)H + 33) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    const int threads = H <= 256 ? 64 : H <= 512 ? 128 : 256;
    const SumTerm a = {d0, w0, k0, e0, s0}, b = {d1, w1, k1, e1, s1}, c = {d2, w2, k2, e2, s2};
#define SAN_LAUNCH(TA)                                                                                                     \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(sum_add_norm_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        pico_launch((sum_add_norm_kernel<TA>), dim3(R), dim3(threads), smem, stream, x, a, b, c, w, kind, eps, (TA*)out, rows, H); \
    } while (0)
    if (act_dtype == PICO_F32) SAN_LAUNCH(float);
    else if (act_dtype == PICO_BF16) SAN_LAUNCH(bf16);
    else return PICO_ERR_DTYPE;
#undef SAN_LAUNCH
    return pico_launch_status();
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// g [T, n] = gelu_tanh(z [T, n]) * table[token[t], off + j]; a token id -(j + 1) names feedback[j] (a token chosen on the
// device in the step before).  table [V, table_stride] in the activation type.
template <typename TA>
__global__ void gelu_gate_rows_kernel(const TA* __restrict__ z, const TA* __restrict__ table, int table_stride, int off,
                                      const int* __restrict__ tokens, const int* __restrict__ feedback, int V, int n,
                                      size_t total, TA* __restrict__ g) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int j = (int)(idx - t * n);
        int id = tokens[t];
        if (id < 0 && feedback) id = feedback[-id - 1];
        id = min(max(id, 0), V - 1);
        g[idx] = from_f32<TA>(gelu_tanh(to_f32(z[idx])) * to_f32(table[(size_t)id * table_stride + off + j]));
    }
}

PICO_API int pico_gelu_gate_rows(const void* z, const void* table, int table_stride, int off, const int* tokens,
                                 const int* feedback, int V, int T, int n, void* g, int dtype, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const size_t total = (size_t)T * n;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((gelu_gate_rows_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)z, (const float*)table,
                    table_stride, off, tokens, feedback, V, n, total, (float*)g);
    else if (dtype == PICO_BF16)
        pico_launch((gelu_gate_rows_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)z, (const bf16*)table,
                    table_stride, off, tokens, feedback, V, n, total, (bf16*)g);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// gu [n, >= 2 ff (+ 1)] rows of row_stride: gate at 0, up at ff, and (row_gate_col >= 0) one more logit at that column whose
// sigmoid multiplies the whole row.  out [n, ff].
template <typename TA>
__global__ void capped_glu_kernel(const TA* __restrict__ gu, int row_stride, int ff, float limit, float alpha, int row_gate_col,
                                  size_t total, TA* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / ff;
        const int j = (int)(idx - p * ff);
        const TA* row = gu + p * row_stride;
        const float g = fminf(to_f32(row[j]), limit);
        const float u = fminf(fmaxf(to_f32(row[ff + j]), -limit), limit);
        float y = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
        if (row_gate_col >= 0) y *= 1.0f / (1.0f + expf(-to_f32(row[row_gate_col])));
        out[idx] = from_f32<TA>(y);
    }
}

// bfloat16 rows whose parts start at multiples of 8 elements: 16 bytes per access.
__global__ void capped_glu_bf16x8_kernel(const bf16* __restrict__ gu, int row_stride, int ff8, float limit, float alpha,
                                         int row_gate_col, size_t total8, bf16* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t p = idx / ff8;
        const int j = (int)(idx - p * ff8) * 8;
        const bf16* row = gu + p * row_stride;
        const uint4 graw = *reinterpret_cast<const uint4*>(row + j);
        const uint4 uraw = *reinterpret_cast<const uint4*>(row + ff8 * 8 + j);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        const float rg = row_gate_col >= 0 ? 1.0f / (1.0f + expf(-to_f32(row[row_gate_col]))) : 1.0f;
        uint4 res;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
            g.x = fminf(g.x, limit);
            g.y = fminf(g.y, limit);
            u.x = fminf(fmaxf(u.x, -limit), limit);
            u.y = fminf(fmaxf(u.y, -limit), limit);
            o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-alpha * g.x)) * (u.x + 1.0f) * rg,
                                          g.y / (1.0f + expf(-alpha * g.y)) * (u.y + 1.0f) * rg);
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = res;
    }
}

PICO_API int pico_capped_glu(const void* gu, int row_stride, int n, int ff, float limit, float alpha, int row_gate_col, void* out,
                             int dtype, cudaStream_t stream) {
    if (n <= 0 || ff <= 0) return 0;
    const size_t total = (size_t)n * ff;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_BF16 && ff % 8 == 0 && row_stride % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const size_t want8 = (total / 8 + 255) / 256;
        pico_launch(capped_glu_bf16x8_kernel, dim3((int)((long long)want8 > cap ? cap : (long long)want8)), dim3(256), 0, stream,
                    (const bf16*)gu, row_stride, ff / 8, limit, alpha, row_gate_col, total / 8, (bf16*)out);
        return pico_launch_status();
    }
    if (dtype == PICO_F32)
        pico_launch((capped_glu_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)gu, row_stride, ff, limit, alpha,
                    row_gate_col, total, (float*)out);
    else if (dtype == PICO_BF16)
        pico_launch((capped_glu_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, row_stride, ff, limit, alpha,
                    row_gate_col, total, (bf16*)out);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
