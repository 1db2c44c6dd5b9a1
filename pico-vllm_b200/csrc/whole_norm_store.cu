// Queries and keys normed over the whole projection, values normed per head, keys and values into their pages.
//
//   q <- q / sqrt(mean over all heads' elements (q^2) + eps) * w_q      (one root mean square for the H * d numbers of a token)
//   k <- the same over the G * d numbers, with w_k;   v_g <- v_g / sqrt(mean(v_g^2) + eps) per key/value head, no weight
//
// A block per token.  q goes to a buffer of its own with heads of `row` elements (row >= d, dv: the attention kernels want
// one head size for queries, keys and values; the elements beyond d or dv are zeros), k and v to the token's place in the
// pages [pages, G, page_size, row] (slot = page * page_size + offset; -1: not stored).  No positions are encoded here.
// Float32 arithmetic; proj and the outputs in the activation type.
#include "common.cuh"

template <typename TA>
__global__ void __launch_bounds__(256)
whole_norm_store_kernel(const TA* __restrict__ proj, int row_stride, int q_off, int k_off, int v_off,
                        const float* __restrict__ q_w, const float* __restrict__ k_w, float eps, int v_norm,
                        const int* __restrict__ slots, TA* __restrict__ k_pages, TA* __restrict__ v_pages, TA* __restrict__ q_out,
                        int H, int G, int d, int dv, int row, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const TA* pr = proj + t * row_stride;
    const int nq = H * d, nk = G * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = to_f32(pr[q_off + i]); ss += x * x; }
    const float inv_q = q_w ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + eps) : 1.0f;
    for (int i = threadIdx.x; i < H * row; i += blockDim.x) {
        const int h = i / row, e = i - h * row;
        q_out[t * ((size_t)H * row) + i] = from_f32<TA>(e < d ? to_f32(pr[q_off + h * d + e]) * inv_q * (q_w ? q_w[h * d + e] : 1.0f) : 0.f);
    }
    const int slot = slots ? slots[t] : -1;
    if (slot < 0) return;
    ss = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float x = to_f32(pr[k_off + i]); ss += x * x; }
    const float inv_k = k_w ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + eps) : 1.0f;
    const size_t page = slot / page_size, off = slot % page_size;
    for (int i = threadIdx.x; i < G * row; i += blockDim.x) {
        const int g = i / row, e = i - g * row;
        k_pages[((page * G + g) * page_size + off) * row + e] =
            from_f32<TA>(e < d ? to_f32(pr[k_off + g * d + e]) * inv_k * (k_w ? k_w[g * d + e] : 1.0f) : 0.f);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int g = warp; g < G; g += nw) {
        float sv = 0.f;
        for (int e = lane; e < dv; e += 32) { const float x = to_f32(pr[v_off + g * dv + e]); sv += x * x; }
        const float inv_v = v_norm ? 1.0f / sqrtf(warp_sum(sv) / (float)dv + eps) : 1.0f;
        TA* dst = v_pages + ((page * G + g) * page_size + off) * row;
        for (int e = lane; e < row; e += 32) dst[e] = from_f32<TA>(e < dv ? to_f32(pr[v_off + g * dv + e]) * inv_v : 0.f);
    }
}

// q_w float32 [H * d] and k_w float32 [G * d], or nullptr (no norm of that projection); v_norm 0/1; slots int32 [T] or nullptr;
// q_out [T, H * row]; pages [pages, G, page_size, row].
PICO_API int pico_whole_norm_store(const void* proj, int row_stride, int q_off, int k_off, int v_off, const float* q_w,
                                   const float* k_w, float eps, int v_norm, const int* slots, void* k_pages, void* v_pages,
                                   void* q_out, int T, int H, int G, int d, int dv, int row, int page_size, int dtype,
                                   cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H < 1 || G < 1 || d < 1 || dv < 1 || row < d || row < dv || page_size < 1) return PICO_ERR_SIZE;
    if (dtype == PICO_F32)
        pico_launch((whole_norm_store_kernel<float>), dim3(T), dim3(256), 0, stream, (const float*)proj, row_stride, q_off, k_off,
                    v_off, q_w, k_w, eps, v_norm, slots, (float*)k_pages, (float*)v_pages, (float*)q_out, H, G, d, dv, row, page_size);
    else if (dtype == PICO_BF16)
        pico_launch((whole_norm_store_kernel<bf16>), dim3(T), dim3(256), 0, stream, (const bf16*)proj, row_stride, q_off, k_off,
                    v_off, q_w, k_w, eps, v_norm, slots, (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, H, G, d, dv, row, page_size);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
