// Queries, keys and values on their way into paged attention when neighbouring dimensions turn together:
//
//   per head of q and of k:  (x[2i], x[2i+1]) <- (x[2i] cos a - x[2i+1] sin a,  x[2i+1] cos a + x[2i] sin a),
//                            a = position * inv_freq[i],  for 2i < rot_dim; the other dimensions pass
//   then, when asked for:    x <- x / sqrt(mean(x^2) + eps) * w       (over the head's d numbers; w may be absent)
//
// q goes out in the activation type with its heads padded with zeros to `row` elements, k and v (v untouched) into the
// token's place of the pages [pages, kv_heads, page_size, row].  The input is float32 rows (what a short convolution left).
// A warp per head of a token (eight heads a block), the head's numbers in registers.  Angles, rotation and norm are float32.
#include "common.cuh"

#define PR_WARPS 8       // heads a block
#define PR_EPL 8         // elements a lane: heads of up to 256

template <typename TA>
__global__ void __launch_bounds__(PR_WARPS * 32)
pair_rope_norm_store_kernel(const float* __restrict__ x, int x_stride, int q_off, int k_off, int v_off,
                            const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim,
                            int norm, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                            const int* __restrict__ slots, TA* __restrict__ k_pages, TA* __restrict__ v_pages,
                            TA* __restrict__ q_out, int H, int G, int d, int dv, int row, int page_size) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * PR_WARPS + warp;            // a warp per head: queries, then keys, then values
    if (head >= H + 2 * G) return;
    const int pos = positions[t];
    const float* in = x + t * x_stride;
    const int slot = slots ? slots[t] : -1;
    const bool is_q = head < H, is_k = !is_q && head < H + G;
    const int a = is_q ? head : is_k ? head - H : head - H - G;
    TA* dst;
    if (is_q) dst = q_out + (t * H + a) * (size_t)row;
    else {
        if (slot < 0 || pos < 0) return;
        TA* pages = is_k ? k_pages : v_pages;
        dst = pages + (((size_t)(slot / page_size) * G + a) * page_size + slot % page_size) * (size_t)row;
    }
    if (pos < 0) {                                   // a padding row: zeros for the kernels behind
        for (int e = lane; e < row; e += 32) dst[e] = from_f32<TA>(0.f);
        return;
    }
    if (!is_q && !is_k) {
        const float* src = in + v_off + a * dv;
        for (int e = lane; e < row; e += 32) dst[e] = from_f32<TA>(e < dv ? src[e] : 0.f);
        return;
    }
    const float* src = in + (is_q ? q_off : k_off) + a * d;
    float vals[PR_EPL];                              // the lane's elements lane, lane + 32, ... after the rotation
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PR_EPL; ++j) {
        const int e = lane + 32 * j;
        float val = 0.f;
        if (e < d) {
            val = src[e];
            if (e < rot_dim) {
                float sn, cs;
                sincosf((float)pos * inv_freq[e >> 1], &sn, &cs);
                const float other = src[e ^ 1];
                val = (e & 1) ? fmaf(val, cs, other * sn) : fmaf(val, cs, -other * sn);
            }
        }
        vals[j] = val;
        ss = fmaf(val, val, ss);
    }
    const float* w = is_q ? q_w : k_w;
    const float inv = norm ? 1.0f / sqrtf(warp_sum(ss) / (float)d + eps) : 1.0f;
#pragma unroll
    for (int j = 0; j < PR_EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < row) dst[e] = from_f32<TA>(e < d ? vals[j] * inv * (norm && w ? w[e] : 1.0f) : 0.f);
    }
}

PICO_API int pico_pair_rope_norm_store(const float* x, int x_stride, int q_off, int k_off, int v_off, const int* positions,
                                       const float* inv_freq, int rot_dim, int norm, const float* q_w, const float* k_w,
                                       float eps, const int* slots, void* k_pages, void* v_pages, void* q_out, int T, int H,
                                       int G, int d, int dv, int row, int page_size, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H < 1 || G < 1 || d < 1 || dv < 1 || row < d || row < dv || rot_dim < 0 || rot_dim > d || (rot_dim & 1) || page_size < 1 ||
        row > 32 * PR_EPL)
        return PICO_ERR_SIZE;
    const dim3 grid(T, (H + 2 * G + PR_WARPS - 1) / PR_WARPS);
    if (dtype == PICO_F32)
        pico_launch((pair_rope_norm_store_kernel<float>), grid, dim3(PR_WARPS * 32), 0, stream, x, x_stride, q_off, k_off, v_off,
                    positions, inv_freq, rot_dim, norm, q_w, k_w, eps, slots, (float*)k_pages, (float*)v_pages, (float*)q_out,
                    H, G, d, dv, row, page_size);
    else if (dtype == PICO_BF16)
        pico_launch((pair_rope_norm_store_kernel<bf16>), grid, dim3(PR_WARPS * 32), 0, stream, x, x_stride, q_off, k_off, v_off,
                    positions, inv_freq, rot_dim, norm, q_w, k_w, eps, slots, (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, H,
                    G, d, dv, row, page_size);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
