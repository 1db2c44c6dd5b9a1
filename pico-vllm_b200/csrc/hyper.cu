// Several residual streams per token (hyper-connections), and the embedding stage's scale and learned positions.
//
// The residual state of a token is S vectors x_1 .. x_S of the model's width, float32, stored [T, S, D].  A sublayer reads
// one mixture of them and writes to all of them:
//
//   u = sum_s in[s] x_s ;   y = sublayer(norm(u)) ;   x_t <- sum_s mix[s, t] x_s + out[t] * y      (all t from the old x)
//
// hyper_step_kernel does, for one token a block, the write of the sublayer BEFORE (its y is still pending when the next
// sublayer asks for its input) and the read of the next one in one pass: every x_s is read once, updated in registers,
// written back, mixed down to u, and u is RMS-normed (a weight per coordinate) into the activation type.  With a list of
// rows (the model's last norm wants a few rows only) nothing is written back.  in == nullptr mixes with ones: the sum of the
// streams, which is what the model's last norm reads.  Everything is float32.
#include "common.cuh"

#define HC_MAX_STREAMS 8

// V consecutive coordinates a thread (4: 16-byte accesses, when the width is a multiple of four)
template <int V>
__device__ __forceinline__ void hc_load(const float* p, float (&o)[V]) {
    if constexpr (V == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else
        o[0] = *p;
}
template <int V>
__device__ __forceinline__ void hc_load(const bf16* p, float (&o)[V]) {
    if constexpr (V == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    } else
        o[0] = __bfloat162float(*p);
}
template <int V>
__device__ __forceinline__ void hc_store(float* p, const float (&o)[V]) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    else *p = o[0];
}
template <int V>
__device__ __forceinline__ void hc_store(bf16* p, const float (&o)[V]) {
    if constexpr (V == 4) {
        uint2 v;
        *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(o[0], o[1]);
        *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(o[2], o[3]);
        *reinterpret_cast<uint2*>(p) = v;
    } else
        *p = __float2bfloat16_rn(o[0]);
}

template <typename TA, int V>
__global__ void __launch_bounds__(256)
hyper_step_kernel(float* __restrict__ x, const TA* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ outw,
                  const float* __restrict__ inw, const float* __restrict__ norm_w, float eps, TA* __restrict__ h,
                  const int* __restrict__ rows, float* __restrict__ sum_out, int S, int D) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float hu[];   // u [D]
    __shared__ float scratch[33];
    __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_out[HC_MAX_STREAMS], s_in[HC_MAX_STREAMS];
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = y ? outw[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    float* xt = x + t * (size_t)S * D;
    float ss = 0.f;
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float xs[HC_MAX_STREAMS][V];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s) {
            if (s < S) hc_load<V>(xt + (size_t)s * D + d, xs[s]);
            else {
#pragma unroll
                for (int e = 0; e < V; ++e) xs[s][e] = 0.f;
            }
        }
        float u[V];
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = 0.f;
        if (y) {
            float yv[V];
            hc_load<V>(y + t * D + d, yv);
#pragma unroll
            for (int to = 0; to < HC_MAX_STREAMS; ++to) {
                if (to >= S) break;
                float acc[V];
#pragma unroll
                for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
                for (int s = 0; s < HC_MAX_STREAMS; ++s)
                    if (s < S) {
                        const float w = s_mix[s * S + to];
#pragma unroll
                        for (int e = 0; e < V; ++e) acc[e] = fmaf(w, xs[s][e], acc[e]);
                    }
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    acc[e] = fmaf(s_out[to], yv[e], acc[e]);
                    u[e] = fmaf(s_in[to], acc[e], u[e]);
                }
                if (!rows) hc_store<V>(xt + (size_t)to * D + d, acc);
            }
        } else {
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) {
#pragma unroll
                    for (int e = 0; e < V; ++e) u[e] = fmaf(s_in[s], xs[s][e], u[e]);
                }
        }
        hc_store<V>(hu + d, u);
#pragma unroll
        for (int e = 0; e < V; ++e) ss += u[e] * u[e];
    }
    // every thread reads back the coordinates it wrote itself: no barrier is needed before these loops
    if (sum_out)
        for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
            float u[V];
            hc_load<V>(hu + d, u);
            hc_store<V>(sum_out + (size_t)r * D + d, u);
        }
    if (!h) return;
    float inv = 1.0f;
    if (norm_w) inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)D + eps);
    for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
        float u[V], w[V];
        hc_load<V>(hu + d, u);
        if (norm_w) {
            hc_load<V>(norm_w + d, w);
#pragma unroll
            for (int e = 0; e < V; ++e) u[e] = u[e] * inv * w[e];
        }
        hc_store<V>(h + (size_t)r * D + d, u);
    }
}

// x float32 [T, S, D] (updated in place unless rows is given); y [T, D] in the activation type or nullptr (nothing pending);
// mix float32 [S, S] (from, to), outw float32 [S]; inw float32 [S] or nullptr (ones); norm_w float32 [D] or nullptr (no norm);
// h [R, D] in the activation type or nullptr; rows int32 [R] or nullptr (R = T); sum_out float32 [R, D] or nullptr (u itself).
PICO_API int pico_hyper_step(float* x, const void* y, const float* mix, const float* outw, const float* inw,
                             const float* norm_w, float eps, void* h, const int* rows, float* sum_out, int R, int S, int D,
                             int dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS || D < 1 || (size_t)D * sizeof(float) > 160 * 1024) return PICO_ERR_SIZE;
    if (y && (!mix || !outw)) return PICO_ERR_SIZE;
    const size_t smem = (size_t)D * sizeof(float);
#define HC_LAUNCH_V(TA, V)                                                                                              \
    do {                                                                                                                \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(hyper_step_kernel<TA, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        pico_launch((hyper_step_kernel<TA, V>), dim3(R), dim3(256), smem, stream, x, (const TA*)y, mix, outw, inw, norm_w, eps, \
                    (TA*)h, rows, sum_out, S, D);                                                                       \
    } while (0)
    // 16-byte accesses when every row starts on such a boundary (8 bytes for bfloat16 rows)
    const bool vec = D % 4 == 0 && ((uintptr_t)x | (uintptr_t)norm_w | (uintptr_t)sum_out) % 16 == 0 &&
                     ((uintptr_t)y | (uintptr_t)h) % 16 == 0;
#define HC_LAUNCH(TA) do { if (vec) HC_LAUNCH_V(TA, 4); else HC_LAUNCH_V(TA, 1); } while (0)
    if (dtype == PICO_F32) HC_LAUNCH(float);
    else if (dtype == PICO_BF16) HC_LAUNCH(bf16);
    else return PICO_ERR_DTYPE;
#undef HC_LAUNCH_V
#undef HC_LAUNCH
    return pico_launch_status();
}

// out[t, s, :] = x[t, :] for every stream s: the streams start as copies of the embedding stage's output.
__global__ void hyper_expand_kernel(const float* __restrict__ x, float* __restrict__ out, int S, int D, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / ((size_t)S * D);
        const int d = (int)(idx % D);
        out[idx] = x[t * D + d];
    }
}

PICO_API int pico_hyper_expand(const float* x, float* out, int T, int S, int D, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (S < 1 || D < 1) return PICO_ERR_SIZE;
    const size_t total = (size_t)T * S * D;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    pico_launch(hyper_expand_kernel, dim3((int)((long long)want > cap ? cap : (long long)want)), dim3(256), 0, stream, x, out, S, D,
                total);
    return pico_launch_status();
}

// x[t, :] = x[t, :] * scale + table[positions[t], :]: the scale of the token embedding and a learned vector per position,
// in float32 on the residual stream.  table (any type) nullptr: the scale alone; a negative position (a padding row) gets
// no vector.
template <typename TW>
__global__ void scale_add_rows_kernel(float* __restrict__ x, float scale, const TW* __restrict__ table,
                                      const int* __restrict__ positions, int D, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / D;
        const int d = (int)(idx - t * D);
        float v = x[idx] * scale;
        if (table) {
            const int p = positions[t];
            if (p >= 0) v += to_f32(table[(size_t)p * D + d]);
        }
        x[idx] = v;
    }
}

PICO_API int pico_scale_add_rows(float* x, float scale, const void* table, const int* positions, int T, int D, int table_dtype,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D < 1 || (table && !positions)) return PICO_ERR_SIZE;
    const size_t total = (size_t)T * D;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (table_dtype == PICO_F32)
        pico_launch((scale_add_rows_kernel<float>), dim3(blocks), dim3(256), 0, stream, x, scale, (const float*)table, positions, D, total);
    else if (table_dtype == PICO_BF16)
        pico_launch((scale_add_rows_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, x, scale, (const bf16*)table, positions, D, total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// out = sa * a + sb * b, element by element, in float32: two mixers side by side whose outputs are weighed and summed.
template <typename TA>
__global__ void scaled_sum_kernel(const TA* __restrict__ a, float sa, const TA* __restrict__ b, float sb, TA* __restrict__ out,
                                  size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = from_f32<TA>(fmaf(sa, to_f32(a[idx]), sb * to_f32(b[idx])));
}

PICO_API int pico_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, long long total, int dtype,
                             cudaStream_t stream) {
    if (total <= 0) return 0;
    const long long cap = 16LL * pico_num_sms();
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want > cap ? cap : want);
    if (dtype == PICO_F32)
        pico_launch((scaled_sum_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb,
                    (float*)out, (size_t)total);
    else if (dtype == PICO_BF16)
        pico_launch((scaled_sum_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)a, sa, (const bf16*)b, sb,
                    (bf16*)out, (size_t)total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
