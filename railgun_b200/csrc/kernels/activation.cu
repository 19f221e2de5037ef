// SiLU-mul of the fused gate|up projection: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(z) = z / (1 + exp(-z)) in 32-bit
// (crates/vllm-models/src/llama/architecture.rs:81-85 computes silu(gate) * up
// with two library ops).
#include "common.cuh"

template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gu, A* __restrict__ out, int I, size_t total) {
    pdl_wait();
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + i]);
    const float u = to_f32(gu[t * 2 * I + I + i]);
    out[idx] = from_f32<A>(g / (1.f + expf(-g)) * u);
}

// Eight outputs per thread with 16-byte loads and stores (bfloat16, I % 8 == 0): the plain storage reads
// gate[i..i+7] and up[i..i+7], the interleaved one reads one 16-column block [8 gate | 8 up].
template <bool INTERLEAVED>
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, size_t groups) {
    pdl_wait();
    pdl_trigger();
    const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gidx >= groups) return;
    const int per_row = I >> 3;
    const size_t t = gidx / per_row;
    const int b = (int)(gidx - t * per_row);
    const bf16* row = gu + t * 2 * (size_t)I;
    const uint4 gv = *reinterpret_cast<const uint4*>(row + (INTERLEAVED ? b * 16 : b * 8));
    const uint4 uv = *reinterpret_cast<const uint4*>(row + (INTERLEAVED ? b * 16 + 8 : I + b * 8));
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        o2[i] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)I + b * 8) = ov;
}

static bool vec8_ok(const void* gu, const void* out, int I) {
    return I % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0;
}

// The same over the interleaved storage of gate|up (rows 16t..16t+7 gate, 16t+8..16t+15 the matching up
// rows), as the decode GEMM's fused epilogue reads it: out[t, 8b + j] = silu(gu[t, 16b + j]) * gu[t, 16b + 8 + j].
template <typename A>
__global__ void silu_mul_interleaved_kernel(const A* __restrict__ gu, A* __restrict__ out, int I, size_t total) {
    pdl_wait();
    pdl_trigger();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const int src = (i >> 3) * 16 + (i & 7);
    const float g = to_f32(gu[t * 2 * I + src]);
    const float u = to_f32(gu[t * 2 * I + src + 8]);
    out[idx] = from_f32<A>(g / (1.f + expf(-g)) * u);
}

extern "C" int rg_silu_mul_interleaved(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    if (I % 8) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    if (dtype == RG_DTYPE_BF16 && vec8_ok(gu, out, I)) {
        const size_t groups = total / 8;
        return rg_launch(silu_mul_vec8_kernel<true>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads),
                         0, s, 1, (const bf16*)gu, (bf16*)out, I, groups);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(silu_mul_interleaved_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu,
                         (bf16*)out, I, total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(silu_mul_interleaved_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu,
                         (float*)out, I, total);
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_silu_mul(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    if (dtype == RG_DTYPE_BF16 && vec8_ok(gu, out, I)) {
        const size_t groups = total / 8;
        return rg_launch(silu_mul_vec8_kernel<false>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads),
                         0, s, 1, (const bf16*)gu, (bf16*)out, I, groups);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)gu, (bf16*)out, I,
                         total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)gu, (float*)out, I,
                         total);
    return RG_ERR_UNSUPPORTED;
}

// Soft cap of logits, in place: z <- cap * tanh(z / cap), 32-bit.
__global__ void softcap_kernel(float* __restrict__ z, float cap, size_t n) {
    pdl_wait();
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

extern "C" int rg_softcap(float* z, float cap, long long n, void* stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    return rg_launch(softcap_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0,
                     (cudaStream_t)stream, 1, z, cap, (size_t)n);
}

// Elementwise activations of a dense feed-forward, computed in 32-bit: 0 relu(z)^2, 1 relu, 2 gelu (tanh form), 3 silu.
__device__ __forceinline__ float act_apply(float z, int kind) {
    switch (kind) {
        case 0: { const float r = fmaxf(z, 0.f); return r * r; }
        case 1: return fmaxf(z, 0.f);
        case 2: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        default: return z / (1.f + expf(-z));
    }
}

template <typename A>
__global__ void activation_kernel(const A* __restrict__ in, A* __restrict__ out, int kind, size_t n) {
    pdl_wait();
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<A>(act_apply(to_f32(in[i]), kind));
}

// Eight bfloat16 numbers per thread with 16-byte loads and stores.
__global__ void activation_vec8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int kind, size_t groups) {
    pdl_wait();
    pdl_trigger();
    const size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const uint4 v = *reinterpret_cast<const uint4*>(in + g * 8);
    const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(v2[i]);
        o2[i] = __floats2bfloat162_rn(act_apply(f.x, kind), act_apply(f.y, kind));
    }
    *reinterpret_cast<uint4*>(out + g * 8) = o;
}

extern "C" int rg_activation(const void* in, void* out, int dtype, int kind, long long n, void* stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 3) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    if (dtype == RG_DTYPE_BF16 && n % 8 == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t groups = (size_t)n / 8;
        return rg_launch(activation_vec8_kernel, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads), 0, s, 1,
                         (const bf16*)in, (bf16*)out, kind, groups);
    }
    const unsigned blocks = (unsigned)(((size_t)n + threads - 1) / threads);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(activation_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, 1, (const bf16*)in, (bf16*)out, kind,
                         (size_t)n);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(activation_kernel<float>, dim3(blocks), dim3(threads), 0, s, 1, (const float*)in, (float*)out, kind,
                         (size_t)n);
    return RG_ERR_UNSUPPORTED;
}

// [T, 2 I] = gate | up  ->  [T, I] = act(gate) * up, for the gated activations of common.cuh (gated_act).
template <typename A>
__global__ void gated_activation_kernel(const A* __restrict__ gu, A* __restrict__ out, int I, int kind, float limit,
                                        size_t total) {
    pdl_wait();
    pdl_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I, i = idx - t * I;
    out[idx] = from_f32<A>(gated_act(to_f32(gu[t * 2 * I + i]), to_f32(gu[t * 2 * I + I + i]), kind, limit));
}

// The same for bfloat16 rows whose halves start on 16-byte boundaries: eight numbers per thread.
__global__ void gated_activation8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I8, int kind,
                                         float limit, size_t total8) {
    pdl_wait();
    pdl_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const size_t t = idx / I8, i = idx - t * I8;
    const uint4 g4 = reinterpret_cast<const uint4*>(gu)[t * 2 * I8 + i];
    const uint4 u4 = reinterpret_cast<const uint4*>(gu)[t * 2 * I8 + I8 + i];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
        o2[j] = __floats2bfloat162_rn(gated_act(g.x, u.x, kind, limit), gated_act(g.y, u.y, kind, limit));
    }
    reinterpret_cast<uint4*>(out)[idx] = o4;
}

extern "C" int rg_gated_activation(const void* gu, void* out, int dtype, int T, int I, int kind, float limit,
                                   void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (kind < 0 || kind > 2) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    if (dtype == RG_DTYPE_BF16 && I % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const size_t total8 = total / 8;
        return rg_launch(gated_activation8_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, s, 1,
                         (const bf16*)gu, (bf16*)out, I / 8, kind, limit, total8);
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(gated_activation_kernel<bf16>, dim3(blocks), dim3(256), 0, s, 1, (const bf16*)gu, (bf16*)out, I,
                         kind, limit, total);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(gated_activation_kernel<float>, dim3(blocks), dim3(256), 0, s, 1, (const float*)gu, (float*)out, I,
                         kind, limit, total);
    return RG_ERR_UNSUPPORTED;
}
