// What grouped-query attention with a norm on q and k does per token before the attention kernels run:
//
//   q_h, k_g <- rotate(w * unit(q_h)), rotate(w * unit(k_g))     unit = divided by its root mean square, either over the
//                                                                d numbers of the head (one weight vector [d] for all q
//                                                                heads, one for all k heads) or, "whole", over all H d
//                                                                numbers of q and all G d of k (weights of that size)
//   rotation of the first `dims` numbers of a head in pairs (2i, 2i + 1) ("interleaved") or (i, i + dims / 2):
//   (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq[i]
//   q_h <- q_h * factor[h] * (1 + coef ln(floor((position + 1) / every) + 1))
//                                                                the score's scale and a number per head, folded in,
//                                                                and a factor that grows with the position (every > 0)
//
// q goes to q_out [T, H, D]; k and v go to the token's place in ordinary key/value pages
// [pages, 2, G, page_size, D].  D >= max(d, dv): keys, queries and values are padded with zeros to one common
// size, so that the paged attention kernels (which know one head size) serve keys and values of different
// sizes; q . k does not notice zeros that q and k share, and the padded output columns are zero.
// Norm, angles, rotation and factors are 32-bit; one rounding into the storage type, which may be narrower than
// the rows' (32-bit rows from a convolution, bfloat16 queries and pages).
#include "common.cuh"

// qkv row: [H * d | G * d | G * dv].
template <typename A, typename O>
__global__ void attention_prepare_kernel(const A* __restrict__ qkv, int ld, O* __restrict__ q_out, O* __restrict__ kv,
                                         const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                         int norm_whole, float eps,
                                         const double* __restrict__ freq, int dims, int interleaved,
                                         const int* __restrict__ positions, const int* __restrict__ slots,
                                         const float* __restrict__ factor, float temp_coef, int temp_every,
                                         int H, int G, int d, int dv, int D, int page_size) {
    extern __shared__ float sm[];                    // cos | sin of the token's dims / 2 angles, then one head's numbers per warp
    __shared__ float whole[2][33];
    float* cs = sm;
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = dims >> 1;
    const int ipos = positions[t];
    const double pos = (double)ipos;
    for (int i = threadIdx.x; i < half; i += blockDim.x) rotary_cos_sin(pos, freq[i], &cs[i], &cs[half + i]);
    const A* row = qkv + (size_t)t * ld;
    float inv_whole_q = 1.f, inv_whole_k = 1.f;
    if (norm_whole && q_norm) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < H * d; i += blockDim.x) { const float v = to_f32(row[i]); sq += v * v; }
        for (int i = threadIdx.x; i < G * d; i += blockDim.x) { const float v = to_f32(row[(size_t)H * d + i]); sk += v * v; }
        sq = block_sum(sq, whole[0]);
        sk = block_sum(sk, whole[1]);
        inv_whole_q = rsqrtf(sq / (float)(H * d) + eps);
        inv_whole_k = rsqrtf(sk / (float)(G * d) + eps);
    }
    __syncthreads();
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((ipos + 1) / temp_every) + 1.f) : 1.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* buf = sm + dims + warp * d;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
    O* kpage = kv + (size_t)page * 2 * G * page_size * D;
    for (int hh = warp; hh < H + G; hh += nwarp) {
        const bool is_q = hh < H;
        if (!is_q && slot < 0) continue;
        const A* src = row + (size_t)hh * d;
        const float* w = is_q ? q_norm : k_norm;
        if (w && norm_whole) w += (size_t)(is_q ? hh : hh - H) * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) { const float v = to_f32(src[i]); buf[i] = v; ss += v * v; }
        ss = warp_sum(ss);
        const float inv = !w ? 1.f : (norm_whole ? (is_q ? inv_whole_q : inv_whole_k) : rsqrtf(ss / (float)d + eps));
        const float f = is_q ? (factor ? factor[hh] : 1.f) * temp : 1.f;
        __syncwarp();
        O* dst = is_q ? q_out + ((size_t)t * H + hh) * D
                      : kpage + ((size_t)(hh - H) * page_size + off) * D;
        for (int i = lane; i < D; i += 32) {
            float v = 0.f;
            if (i < d) {
                v = buf[i] * inv * (w ? w[i] : 1.f);
                if (i < dims) {
                    int mate, a;
                    bool first;
                    if (interleaved) { first = (i & 1) == 0; mate = i ^ 1; a = i >> 1; }
                    else { first = i < half; mate = first ? i + half : i - half; a = first ? i : i - half; }
                    const float m = buf[mate] * inv * (w ? w[mate] : 1.f);
                    v = first ? v * cs[a] - m * cs[half + a] : v * cs[a] + m * cs[half + a];
                }
                v *= f;
            }
            dst[i] = from_f32<O>(v);
        }
        __syncwarp();
    }
    if (slot >= 0) {
        const A* vsrc = row + (size_t)(H + G) * d;
        O* vpage = kpage + (size_t)G * page_size * D;
        for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
            const int g = e / D, i = e - g * D;
            vpage[((size_t)g * page_size + off) * D + i] = from_f32<O>(i < dv ? to_f32(vsrc[(size_t)g * dv + i]) : 0.f);
        }
    }
}

extern "C" int rg_attention_prepare(const void* qkv, int dtype, int ld, void* q_out, int out_dtype, void* kv,
                                    const float* q_norm, const float* k_norm, int norm_whole, float eps,
                                    const double* freq, int dims, int interleaved,
                                    const int* positions, const int* slots, const float* factor, float temp_coef,
                                    int temp_every, int T, int H, int G, int d, int dv, int D, int page_size,
                                    void* stream) {
    if (T <= 0) return 0;
    if (dims < 0 || dims > d || (dims & 1) || H < 1 || G < 1 || H % G || d < 1 || dv < 1 || D < d || D < dv || page_size < 1
        || (q_norm == nullptr) != (k_norm == nullptr) || temp_every < 0)
        return RG_ERR_UNSUPPORTED;
    int nwarp = H + G < 16 ? H + G : 16;
    if (nwarp < 4) nwarp = 4;
    while (nwarp > 4 && (size_t)(dims + nwarp * d) * sizeof(float) > 40 * 1024) --nwarp;
    const size_t smem = (size_t)(dims + nwarp * d) * sizeof(float);
    if (smem > 40 * 1024) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define RG_PREPARE(A, O) return rg_launch(attention_prepare_kernel<A, O>, dim3(T), dim3(32 * nwarp), smem, s, 1, \
        (const A*)qkv, ld, (O*)q_out, (O*)kv, q_norm, k_norm, norm_whole, eps, freq, dims, interleaved, positions, slots, \
        factor, temp_coef, temp_every, H, G, d, dv, D, page_size)
    if (dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) RG_PREPARE(bf16, bf16);
    if (dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) RG_PREPARE(float, float);
    if (dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) RG_PREPARE(float, bf16);
#undef RG_PREPARE
    return RG_ERR_UNSUPPORTED;
}
