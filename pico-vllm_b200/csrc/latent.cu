// Kernels of the latent-attention mixer: what stands between its matrix products.
//
// A token's down projection row holds, side by side, the query latent (q_rank; 0: the queries are projected directly), the key/value latent
// (kv_rank; absent in a layer that reads another layer's cache) and one gate logit per head.
// latent_norm_store_kernel, one block of three warps per token (a warp per part):
//   c_q  = u_q / sqrt(mean(u_q^2) + eps) * w_q                -> cq [T, q_rank]       (activation type)
//   c    = u_kv / sqrt(mean(u_kv^2) + eps) * w_kv             -> the token's cache row (cache type), zero
//                                                                beyond kv_rank up to the row's width
//   gate = 1 / (1 + exp(-u_g))                                -> gate [T, heads]      (float32)
// All arithmetic in float32.  A token whose slot is negative stores nothing (padding rows).
//
// head_scale_kernel: o[t, h, :] *= gate[t, h]  (the per-head output gate).
#include "common.cuh"

// One warp per part of the row (query latent, key/value latent, gates): sums through shuffles, no block barrier.
template <typename TA>
__device__ __forceinline__ void rms_part(const TA* __restrict__ src, int n, const float* __restrict__ w, float eps,
                                         TA* __restrict__ dst, int dst_n, int lane) {
    float ss = 0.f;
#pragma unroll 8
    for (int i = lane; i < n; i += 32) {
        const float v = to_f32(src[i]);
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
#pragma unroll 8
    for (int i = lane; i < dst_n; i += 32) dst[i] = i < n ? from_f32<TA>(to_f32(src[i]) * inv * w[i]) : from_f32<TA>(0.f);
}

template <typename TA>
__global__ void __launch_bounds__(96) latent_norm_store_kernel(const TA* __restrict__ proj, int proj_stride, int q_off,
                                                               int q_rank, const float* __restrict__ wq, TA* __restrict__ cq,
                                                               int kv_off, int kv_rank, const float* __restrict__ wkv,
                                                               const int* __restrict__ slots, TA* __restrict__ cache,
                                                               int cache_row, int g_off, int heads,
                                                               float* __restrict__ gate, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TA* row = proj + (size_t)t * proj_stride;
    if (warp == 0) {
        if (q_rank > 0) rms_part<TA>(row + q_off, q_rank, wq, eps, cq + (size_t)t * q_rank, q_rank, lane);
    } else if (warp == 1) {
        const int slot = kv_rank > 0 && slots ? slots[t] : -1;
        if (slot >= 0) rms_part<TA>(row + kv_off, kv_rank, wkv, eps, cache + (size_t)slot * cache_row, cache_row, lane);
    } else {
        for (int h = lane; h < heads; h += 32)
            gate[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-to_f32(row[g_off + h])));
    }
}

// proj [T, >= all offsets] with row stride proj_stride; cq [T, q_rank]; cache rows of cache_row elements
// (>= kv_rank); slots int32 [T] or nullptr with kv_rank 0; gate float32 [T, heads].
PICO_API int pico_latent_norm_store(const void* proj, int proj_stride, int q_off, int q_rank, const float* wq, void* cq,
                                    int kv_off, int kv_rank, const float* wkv, const int* slots, void* cache,
                                    int cache_row, int g_off, int heads, float* gate, float eps, int T, int dtype,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_rank < 0 || heads < 0 || kv_rank < 0 || (q_rank > 0 && (!wq || !cq)) || (heads > 0 && !gate) || (kv_rank > 0 && (cache_row < kv_rank || !cache || !wkv)))
        return PICO_ERR_SIZE;
    const int threads = 96;
    if (dtype == PICO_F32)
        pico_launch((latent_norm_store_kernel<float>), dim3(T), dim3(threads), 0, stream, (const float*)proj, proj_stride,
                    q_off, q_rank, wq, (float*)cq, kv_off, kv_rank, wkv, slots, (float*)cache, cache_row, g_off, heads,
                    gate, eps);
    else if (dtype == PICO_BF16)
        pico_launch((latent_norm_store_kernel<bf16>), dim3(T), dim3(threads), 0, stream, (const bf16*)proj, proj_stride,
                    q_off, q_rank, wq, (bf16*)cq, kv_off, kv_rank, wkv, slots, (bf16*)cache, cache_row, g_off, heads,
                    gate, eps);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// VEC: head_width a multiple of 8 (bfloat16) or 4 (float32): 16 bytes per access.
template <typename TA, bool VEC>
__global__ void head_scale_kernel(TA* __restrict__ o, const float* __restrict__ gate, int head_width, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int W = VEC ? 16 / (int)sizeof(TA) : 1;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t at = idx * W;
        const float g = gate[at / head_width];
        if (VEC) {
            uint4 raw = *reinterpret_cast<const uint4*>(o + at);
            TA* v = reinterpret_cast<TA*>(&raw);
#pragma unroll
            for (int k = 0; k < W; ++k) v[k] = from_f32<TA>(to_f32(v[k]) * g);
            *reinterpret_cast<uint4*>(o + at) = raw;
        } else {
            o[at] = from_f32<TA>(to_f32(o[at]) * g);
        }
    }
}

// o [T, heads * head_width] contiguous, gate float32 [T, heads]: o[t, h, :] *= gate[t, h].
PICO_API int pico_head_scale(void* o, const float* gate, int T, int heads, int head_width, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || head_width <= 0) return PICO_ERR_SIZE;
    if (dtype != PICO_F32 && dtype != PICO_BF16) return PICO_ERR_DTYPE;
    const int w = dtype == PICO_F32 ? 4 : 8;
    const bool vec = head_width % w == 0;
    const size_t total = (size_t)T * heads * head_width / (vec ? w : 1);
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32) {
        if (vec) pico_launch((head_scale_kernel<float, true>), dim3(blocks), dim3(256), 0, stream, (float*)o, gate, head_width, total);
        else pico_launch((head_scale_kernel<float, false>), dim3(blocks), dim3(256), 0, stream, (float*)o, gate, head_width, total);
    } else {
        if (vec) pico_launch((head_scale_kernel<bf16, true>), dim3(blocks), dim3(256), 0, stream, (bf16*)o, gate, head_width, total);
        else pico_launch((head_scale_kernel<bf16, false>), dim3(blocks), dim3(256), 0, stream, (bf16*)o, gate, head_width, total);
    }
    return pico_launch_status();
}
