// Fused residual-add + RMSNorm.
//
//   r = residual[row] (+ pending[row])        32-bit sum, written back
//   out[i] = w * r / sqrt(mean(r^2) + eps)     sum of squares, rsqrt and the
//                                              product in 32-bit, one rounding
// The reference builds the norm from its tensor library
// (crates/vllm-models/src/llama/architecture.rs:27-28,48,56,154) and adds the
// residual as a separate op (:53,58); here both are one pass over the row.
// With `rows` given, output row i is computed from residual row rows[i] and the
// residual is not written back (the final norm runs only where logits are wanted).
#include "common.cuh"

template <typename P, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const P* __restrict__ pending,
                                   const float* __restrict__ w, float eps, O* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const P* p = pending ? pending + (size_t)srow * H : nullptr;
    const bool write_back = (rows == nullptr) && (p != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p) v += to_f32(p[i]);
        if (write_back) r[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    O* o = out + (size_t)orow * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p && !write_back) v += to_f32(p[i]);
        o[i] = from_f32<O>(v * inv * w[i]);
    }
}

// The same with 4 elements per access for H % 4 == 0 (16-byte residual accesses).  The order of the sum of
// squares inside a thread differs from the scalar kernel's, the block reduction is the same.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}

template <typename P, typename O>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ resid, const P* __restrict__ pending,
                                        const float* __restrict__ w, float eps, O* __restrict__ out,
                                        const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const P* p = pending ? pending + (size_t)srow * H : nullptr;
    const bool write_back = (rows == nullptr) && (p != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = load4(r + i);
        if (p) {
            const float4 q = load4(p + i);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
            if (write_back) store4(r + i, v);
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    O* o = out + (size_t)orow * H;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        float4 v = load4(r + i);
        if (p && !write_back) {
            const float4 q = load4(p + i);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
        const float4 g = load4(w + i);
        store4(o + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
    }
}

// residual[row] += pending[row] only (a block arrangement that ends without a norm).
template <typename P>
__global__ void residual_add_kernel(float* __restrict__ resid, const P* __restrict__ pending, size_t n) {
    pdl_wait();
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += to_f32(pending[i]);
}

extern "C" int rg_add_rmsnorm(float* resid, const void* pending, int pending_dtype, const float* w,
                              float eps, void* out, int out_dtype, const int* rows, int n_out_rows,
                              int H, void* stream) {
    if (n_out_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (uintptr_t)pending % 16 == 0 && (uintptr_t)w % 16 == 0;
    const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define RG_NORM(P, O) return vec ? rg_launch(add_rmsnorm_vec4_kernel<P, O>, dim3(n_out_rows), dim3(threads), 0, s, 1, \
        resid, (const P*)pending, w, eps, (O*)out, rows, H) \
      : rg_launch(add_rmsnorm_kernel<P, O>, dim3(n_out_rows), dim3(threads), 0, s, 1, \
        resid, (const P*)pending, w, eps, (O*)out, rows, H)
    if (pending == nullptr) pending_dtype = out_dtype;
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) RG_NORM(bf16, bf16);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) RG_NORM(float, float);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) RG_NORM(float, bf16);
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_F32) RG_NORM(bf16, float);
#undef RG_NORM
    return RG_ERR_UNSUPPORTED;
}

// The residual step of a block with a norm behind each part as well as before it:
//   u = post_w * y / sqrt(mean(y^2) + post_eps)    the part's output y, normed (post_w holds the norm's weight
//                                                  with whatever constant factors follow it multiplied in)
//   r = residual[row] + u                          32-bit, written back
//   out = w * r / sqrt(mean(r^2) + eps)            the next part's input; with w == nullptr out = r, unnormed
//                                                  (a copy of the stream in the activation type); out == nullptr: none
// Both sums of squares, both roots and the additions are 32-bit; y is read twice (the second read hits L1/L2).
// post_w == nullptr adds y as it is.  `rows` as in add_rmsnorm_kernel.  out rows are out_ld elements apart.
template <typename P, typename O>
__global__ void add_postnorm_rmsnorm_kernel(float* __restrict__ resid, const P* __restrict__ pending,
                                            const float* __restrict__ post_w, float post_eps,
                                            const float* __restrict__ w, float eps, O* __restrict__ out, int out_ld,
                                            const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const P* p = pending ? pending + (size_t)srow * H : nullptr;
    float inv_y = 1.f;
    if (p && post_w) {
        float sy = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) { const float y = to_f32(p[i]); sy += y * y; }
        sy = block_sum(sy, scratch);
        inv_y = rsqrtf(sy / (float)H + post_eps);
    }
    const bool write_back = (rows == nullptr) && (p != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p) v += post_w ? to_f32(p[i]) * inv_y * post_w[i] : to_f32(p[i]);
        if (write_back) r[i] = v;
        ss += v * v;
    }
    if (out == nullptr) return;
    float inv = 1.f;
    if (w) {
        ss = block_sum(ss, scratch);
        inv = rsqrtf(ss / (float)H + eps);
    } else {
        __syncthreads();
    }
    O* o = out + (size_t)orow * out_ld;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = r[i];
        if (p && !write_back) v += post_w ? to_f32(p[i]) * inv_y * post_w[i] : to_f32(p[i]);
        o[i] = from_f32<O>(w ? v * inv * w[i] : v);
    }
}

extern "C" int rg_add_postnorm_rmsnorm(float* resid, const void* pending, int pending_dtype, const float* post_w,
                                       float post_eps, const float* w, float eps, void* out, int out_dtype,
                                       int out_ld, const int* rows, int n_out_rows, int H, void* stream) {
    if (n_out_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define RG_PNORM(P, O) return rg_launch(add_postnorm_rmsnorm_kernel<P, O>, dim3(n_out_rows), dim3(threads), 0, s, 1, \
        resid, (const P*)pending, post_w, post_eps, w, eps, (O*)out, out_ld, rows, H)
    if (pending == nullptr) pending_dtype = RG_DTYPE_F32;
    if (out == nullptr) out_dtype = RG_DTYPE_F32;
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) RG_PNORM(bf16, bf16);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) RG_PNORM(float, float);
    if (pending_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) RG_PNORM(float, bf16);
    if (pending_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_F32) RG_PNORM(bf16, float);
#undef RG_PNORM
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_residual_add(float* resid, const void* pending, int pending_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (pending_dtype == RG_DTYPE_BF16)
        return rg_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, resid, (const bf16*)pending,
                         (size_t)n);
    if (pending_dtype == RG_DTYPE_F32)
        return rg_launch(residual_add_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, resid, (const float*)pending,
                         (size_t)n);
    return RG_ERR_UNSUPPORTED;
}

// RMSNorm in groups after up to two additions, with up to two weights (a block whose mixer and feed-forward
// read the same stream, each through a norm of its own):
//   r = residual[row] + (p1[row] + p2[row])                 32-bit, written back (not with `rows`)
//   the row is cut into `groups` equal consecutive parts; each part is divided by its own sqrt(mean(part^2) + eps)
//   out_k = w_k * that, k = 1, 2 (out2 may be absent)
// The block's eight warps form teams of 8 / groups warps (at least one), a team per group at a time; a team adds
// its squares in a fixed order, so a row's result does not depend on what else is in the step.
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == RG_DTYPE_BF16 ? __bfloat162float(reinterpret_cast<const bf16*>(p)[i])
                                  : reinterpret_cast<const float*>(p)[i];
}

template <typename O>
__global__ void __launch_bounds__(256) add_group_rmsnorm_kernel(
        float* __restrict__ resid, const void* __restrict__ p1, int p1_dtype, const void* __restrict__ p2, int p2_dtype,
        const float* __restrict__ w1, const float* __restrict__ w2, float eps, O* __restrict__ out1,
        O* __restrict__ out2, const int* __restrict__ rows, int H, int groups, int wpt) {
    __shared__ float scratch[8];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const size_t pbase = (size_t)srow * H;
    const bool write_back = rows == nullptr && (p1 != nullptr || p2 != nullptr);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nteams = 8 / wpt, team = warp / wpt, in_team = (warp - team * wpt) * 32 + lane, team_threads = wpt * 32;
    const int gs = H / groups;
    for (int g0 = 0; g0 < groups; g0 += nteams) {
        const int g = g0 + team;
        const bool active = g < groups;
        const int lo = g * gs;
        float ss = 0.f;
        if (active) {
            for (int i = lo + in_team; i < lo + gs; i += team_threads) {
                float v = r[i];
                if (p1 || p2) {
                    float add = p1 ? load_any(p1, p1_dtype, pbase + i) : 0.f;
                    if (p2) add += load_any(p2, p2_dtype, pbase + i);
                    v += add;
                    if (write_back) r[i] = v;
                }
                ss += v * v;
            }
        }
        ss = warp_sum(ss);
        if (wpt > 1) {
            if (lane == 0) scratch[warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int k = 0; k < wpt; ++k) ss += scratch[team * wpt + k];
            __syncthreads();
        }
        if (!active) continue;
        const float inv = rsqrtf(ss / (float)gs + eps);
        for (int i = lo + in_team; i < lo + gs; i += team_threads) {
            float v = r[i];
            if (!write_back && (p1 || p2)) {
                float add = p1 ? load_any(p1, p1_dtype, pbase + i) : 0.f;
                if (p2) add += load_any(p2, p2_dtype, pbase + i);
                v += add;
            }
            v *= inv;
            out1[(size_t)orow * H + i] = from_f32<O>(v * w1[i]);
            if (out2) out2[(size_t)orow * H + i] = from_f32<O>(v * w2[i]);
        }
    }
}

// The same with four numbers per thread and step (16-byte accesses to the 32-bit rows, 8-byte ones to bfloat16
// rows), where the groups' sizes and the addresses allow it.
__device__ __forceinline__ float4 load_any4(const void* p, int dtype, size_t i) {
    if (dtype == RG_DTYPE_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
}

template <typename O>
__global__ void __launch_bounds__(256) add_group_rmsnorm4_kernel(
        float* __restrict__ resid, const void* __restrict__ p1, int p1_dtype, const void* __restrict__ p2, int p2_dtype,
        const float* __restrict__ w1, const float* __restrict__ w2, float eps, O* __restrict__ out1,
        O* __restrict__ out2, const int* __restrict__ rows, int H, int groups, int wpt) {
    __shared__ float scratch[8];
    pdl_wait();
    pdl_trigger();
    const int orow = blockIdx.x;
    const int srow = rows ? rows[orow] : orow;
    float* r = resid + (size_t)srow * H;
    const size_t pbase = (size_t)srow * H;
    const bool write_back = rows == nullptr && (p1 != nullptr || p2 != nullptr);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nteams = 8 / wpt, team = warp / wpt, in_team = (warp - team * wpt) * 32 + lane, team_threads = wpt * 32;
    const int gs = H / groups, gs4 = gs >> 2;
    for (int g0 = 0; g0 < groups; g0 += nteams) {
        const int g = g0 + team;
        const bool active = g < groups;
        const int lo = g * gs;
        float ss = 0.f;
        if (active) {
            for (int i4 = in_team; i4 < gs4; i4 += team_threads) {
                const int i = lo + 4 * i4;
                float4 v = *reinterpret_cast<const float4*>(r + i);
                if (p1 || p2) {
                    if (p1) { const float4 a = load_any4(p1, p1_dtype, pbase + i); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
                    if (p2) { const float4 a = load_any4(p2, p2_dtype, pbase + i); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
                    if (write_back) *reinterpret_cast<float4*>(r + i) = v;
                }
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        ss = warp_sum(ss);
        if (wpt > 1) {
            if (lane == 0) scratch[warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int k = 0; k < wpt; ++k) ss += scratch[team * wpt + k];
            __syncthreads();
        }
        if (!active) continue;
        const float inv = rsqrtf(ss / (float)gs + eps);
        for (int i4 = in_team; i4 < gs4; i4 += team_threads) {
            const int i = lo + 4 * i4;
            float4 v = *reinterpret_cast<const float4*>(r + i);
            if (!write_back && (p1 || p2)) {
                if (p1) { const float4 a = load_any4(p1, p1_dtype, pbase + i); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
                if (p2) { const float4 a = load_any4(p2, p2_dtype, pbase + i); v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
            }
            v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
            const float4 a = *reinterpret_cast<const float4*>(w1 + i);
            store4(out1 + (size_t)orow * H + i, make_float4(v.x * a.x, v.y * a.y, v.z * a.z, v.w * a.w));
            if (out2) {
                const float4 b = *reinterpret_cast<const float4*>(w2 + i);
                store4(out2 + (size_t)orow * H + i, make_float4(v.x * b.x, v.y * b.y, v.z * b.z, v.w * b.w));
            }
        }
    }
}

extern "C" int rg_add_group_rmsnorm(float* resid, const void* p1, int p1_dtype, const void* p2, int p2_dtype,
                                    const float* w1, const float* w2, float eps, void* out1, void* out2, int out_dtype,
                                    const int* rows, int n_out_rows, int H, int groups, void* stream) {
    if (n_out_rows <= 0) return 0;
    if (groups < 1 || H % groups || (out2 && !w2)) return RG_ERR_UNSUPPORTED;
    int wpt = 8;
    while (wpt > 1 && wpt * groups > 8) wpt >>= 1;
    cudaStream_t s = (cudaStream_t)stream;
    auto aligned = [](const void* p, int dtype) { return ((uintptr_t)p & (dtype == RG_DTYPE_BF16 ? 7 : 15)) == 0; };
    if ((H / groups) % 4 == 0 && ((uintptr_t)resid & 15) == 0 && aligned(p1, p1_dtype) && aligned(p2, p2_dtype) &&
        ((uintptr_t)w1 & 15) == 0 && ((uintptr_t)w2 & 15) == 0 && aligned(out1, out_dtype) && aligned(out2, out_dtype)) {
        if (out_dtype == RG_DTYPE_BF16)
            return rg_launch(add_group_rmsnorm4_kernel<bf16>, dim3(n_out_rows), dim3(256), 0, s, 1, resid, p1, p1_dtype,
                             p2, p2_dtype, w1, w2, eps, (bf16*)out1, (bf16*)out2, rows, H, groups, wpt);
        if (out_dtype == RG_DTYPE_F32)
            return rg_launch(add_group_rmsnorm4_kernel<float>, dim3(n_out_rows), dim3(256), 0, s, 1, resid, p1, p1_dtype,
                             p2, p2_dtype, w1, w2, eps, (float*)out1, (float*)out2, rows, H, groups, wpt);
    }
    if (out_dtype == RG_DTYPE_BF16)
        return rg_launch(add_group_rmsnorm_kernel<bf16>, dim3(n_out_rows), dim3(256), 0, s, 1, resid, p1, p1_dtype, p2,
                         p2_dtype, w1, w2, eps, (bf16*)out1, (bf16*)out2, rows, H, groups, wpt);
    if (out_dtype == RG_DTYPE_F32)
        return rg_launch(add_group_rmsnorm_kernel<float>, dim3(n_out_rows), dim3(256), 0, s, 1, resid, p1, p1_dtype, p2,
                         p2_dtype, w1, w2, eps, (float*)out1, (float*)out2, rows, H, groups, wpt);
    return RG_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------
// The sum of several rows, each first RMS-normed with a weight and a constant of its own:
//   out[t] (32-bit) = sum_b c_b * y_b[t] / sqrt(mean(y_b[t]^2) + eps) * w_b
// for branches that run side by side and are brought to one size before they are added.  One block per row;
// a thread keeps its numbers of every input in registers between the two passes (up to NS_KEEP per input).
// ---------------------------------------------------------------------------------------------------
#define NS_MAX 4
#define NS_KEEP 8
struct NormSumArgs {
    const void* y[NS_MAX];
    const float* w[NS_MAX];
    float c[NS_MAX];
    int n;
};

template <typename P>
__global__ void __launch_bounds__(256) norm_sum_kernel(NormSumArgs a, float eps, float* __restrict__ out, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * H;
    float acc[NS_KEEP];
#pragma unroll
    for (int j = 0; j < NS_KEEP; ++j) acc[j] = 0.f;
#pragma unroll
    for (int b = 0; b < NS_MAX; ++b) {
        if (b >= a.n) break;
        const P* y = reinterpret_cast<const P*>(a.y[b]) + base;
        float keep[NS_KEEP];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NS_KEEP; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            keep[j] = i < H ? to_f32(y[i]) : 0.f;
            ss += keep[j] * keep[j];
        }
        for (int i = threadIdx.x + NS_KEEP * blockDim.x; i < H; i += blockDim.x) { const float v = to_f32(y[i]); ss += v * v; }
        ss = block_sum(ss, scratch);
        const float f = rsqrtf(ss / (float)H + eps) * a.c[b];
        const float* w = a.w[b];
#pragma unroll
        for (int j = 0; j < NS_KEEP; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < H) acc[j] += keep[j] * f * w[i];
        }
        for (int i = threadIdx.x + NS_KEEP * blockDim.x; i < H; i += blockDim.x) {
            const float v = to_f32(y[i]) * f * w[i];
            if (b == 0) out[base + i] = v; else out[base + i] += v;
        }
    }
#pragma unroll
    for (int j = 0; j < NS_KEEP; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < H) out[base + i] = acc[j];
    }
}

// The same with 16-byte loads: a thread holds NV pieces of 8 bfloat16 (or 4 float) numbers of every input, rows and
// weights start on 16-byte boundaries, H is a multiple of the piece.
template <typename P, int NV>
__global__ void __launch_bounds__(256) norm_sum_vec_kernel(NormSumArgs a, float eps, float* __restrict__ out, int H) {
    constexpr int PIECE = 16 / sizeof(P);
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * H;
    const int pieces = H / PIECE;
    float acc[NV][PIECE];
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < PIECE; ++e) acc[j][e] = 0.f;
#pragma unroll
    for (int b = 0; b < NS_MAX; ++b) {
        if (b >= a.n) break;
        const P* y = reinterpret_cast<const P*>(a.y[b]) + base;
        float keep[NV][PIECE];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < pieces) {
                const uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)i * PIECE);
                if (sizeof(P) == 2) {
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int e = 0; e < PIECE / 2; ++e) {
                        const float2 f = __bfloat1622float2(h2[e]);
                        keep[j][2 * e] = f.x;
                        keep[j][2 * e + 1] = f.y;
                    }
                } else {
                    const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
                    for (int e = 0; e < PIECE; ++e) keep[j][e] = f[e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < PIECE; ++e) keep[j][e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < PIECE; ++e) ss += keep[j][e] * keep[j][e];
        }
        ss = block_sum(ss, scratch);
        const float f = rsqrtf(ss / (float)H + eps) * a.c[b];
        const float* w = a.w[b];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < pieces) {
#pragma unroll
                for (int e4 = 0; e4 < PIECE / 4; ++e4) {
                    const float4 wv = *reinterpret_cast<const float4*>(w + (size_t)i * PIECE + 4 * e4);
                    acc[j][4 * e4] += keep[j][4 * e4] * f * wv.x;
                    acc[j][4 * e4 + 1] += keep[j][4 * e4 + 1] * f * wv.y;
                    acc[j][4 * e4 + 2] += keep[j][4 * e4 + 2] * f * wv.z;
                    acc[j][4 * e4 + 3] += keep[j][4 * e4 + 3] * f * wv.w;
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < pieces) {
#pragma unroll
            for (int e4 = 0; e4 < PIECE / 4; ++e4)
                *reinterpret_cast<float4*>(out + base + (size_t)i * PIECE + 4 * e4) =
                    make_float4(acc[j][4 * e4], acc[j][4 * e4 + 1], acc[j][4 * e4 + 2], acc[j][4 * e4 + 3]);
        }
    }
}

// ys, ws: n pointers each (rows of H numbers of type `dtype`; weights [H] float); cs: n constants.
extern "C" int rg_norm_sum(const void* const* ys, const float* const* ws, const float* cs, int n, int dtype, float eps,
                           float* out, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (n < 1 || n > NS_MAX || H < 1) return RG_ERR_UNSUPPORTED;
    NormSumArgs a;
    a.n = n;
    uintptr_t bits = (uintptr_t)out;
    for (int b = 0; b < NS_MAX; ++b) {
        a.y[b] = b < n ? ys[b] : nullptr;
        a.w[b] = b < n ? ws[b] : nullptr;
        a.c[b] = b < n ? cs[b] : 0.f;
        if (b < n) bits |= (uintptr_t)ys[b] | (uintptr_t)ws[b];
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int piece = dtype == RG_DTYPE_BF16 ? 8 : 4;
    if ((bits & 15) == 0 && H % piece == 0 && H / piece <= 4 * 256 && (dtype == RG_DTYPE_BF16 || dtype == RG_DTYPE_F32)) {
        const int pieces = H / piece;
        const int nv = pieces <= 256 ? 1 : (pieces <= 512 ? 2 : 4);
        int threads = ((pieces + nv - 1) / nv + 31) / 32 * 32;
        if (threads < 32) threads = 32;
#define RG_NSV(P, NV) return rg_launch(norm_sum_vec_kernel<P, NV>, dim3(T), dim3(threads), 0, s, 1, a, eps, out, H)
        if (dtype == RG_DTYPE_BF16) { if (nv == 1) RG_NSV(bf16, 1); if (nv == 2) RG_NSV(bf16, 2); RG_NSV(bf16, 4); }
        if (nv == 1) RG_NSV(float, 1);
        if (nv == 2) RG_NSV(float, 2);
        RG_NSV(float, 4);
#undef RG_NSV
    }
    const int threads = H >= 2048 ? 256 : (H >= 512 ? 128 : 64);
    if (dtype == RG_DTYPE_BF16) return rg_launch(norm_sum_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, a, eps, out, H);
    if (dtype == RG_DTYPE_F32) return rg_launch(norm_sum_kernel<float>, dim3(T), dim3(threads), 0, s, 1, a, eps, out, H);
    return RG_ERR_UNSUPPORTED;
}
