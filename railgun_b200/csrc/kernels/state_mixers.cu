// Mixers whose memory is a matrix per head instead of a growing cache, and the short causal convolutions
// that sit in front of them.
//
//   causal_conv        y_t = [x_t +] act(sum_j w[:, j] x_(t - K + 1 + j)) per channel, K taps, the last column of w the
//                      current token's; continued from the K - 1 inputs a request keeps in its state slot
//   conv_state_update  leaves the step's last K - 1 inputs in the slot
//   retention_prepare  rotation of q and k in pairs (i, i + dims / 2), k times a constant, into 32-bit rows
//   delta_prepare      q and k to unit length per head (q times a constant), beta = sigmoid(b),
//                      g = exp(-exp(A) softplus(a + bias)) per head
//   state_scan         per head, token by token, S [d, dv] in 32-bit:
//                        retention:  S <- decay_h S + k v^T;                         o = S^T q
//                        delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
//                      (Sun et al., "Retentive Network: A Successor to Transformer for Large Language Models";
//                      Yang et al., "Gated Delta Networks: Improving Mamba2 with Delta Rule")
//   head_norm_gate     o / rms(o) per head [times a weight], times silu(gate), rounded once for the output product
//
// The step's tokens are packed request by request (cu_seqlens); a request whose start position is 0 begins
// from zeros whatever its slot holds; a row whose request has slot -1 (padding of a static batch) reads zeros
// and writes no state.  A token's result depends on its request's earlier tokens only through the state, which
// is carried in 32-bit, so cutting a prompt into portions changes no bit.
#include "common.cuh"

__device__ __forceinline__ float sm_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float sm_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

// x: rows ld apart, channel c at column x_off + c.  taps [K, C] float (tap-major, so that neighbouring channels
// are neighbouring numbers; row K - 1 is the current token's).  state [slots, K - 1, C] float, oldest input first.
// out: rows out_ld apart (type O).  residual: out = x + conv(x); act 1: silu of the convolution.
template <typename A, typename O>
__global__ void causal_conv_kernel(const A* __restrict__ x, int ld, int x_off, const float* __restrict__ taps,
                                   const float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ req_of_token, const int* __restrict__ start_pos,
                                   const int* __restrict__ slots, O* __restrict__ out, int out_ld, int C, int K,
                                   int residual, int act) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r = req_of_token[t];
    const int i = t - cu_seqlens[r];
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
        const int idx = i - (K - 1) + j;                     // the step's token this tap reads; negative: before the step
        float v;
        if (idx >= 0) v = to_f32(x[(size_t)(t - (K - 1) + j) * ld + x_off + c]);
        else v = has_past ? state[((size_t)slot * (K - 1) + (K - 1 + idx)) * C + c] : 0.f;
        acc += taps[(size_t)j * C + c] * v;
    }
    if (act == 1) acc = acc * sm_sigmoid(acc);
    if (residual) acc += to_f32(x[(size_t)t * ld + x_off + c]);
    out[(size_t)t * out_ld + c] = from_f32<O>(acc);
}

// The same for bfloat16 inputs with eight channels per thread (16-byte loads), where rows and offsets allow it.
template <typename O>
__global__ void causal_conv8_kernel(const bf16* __restrict__ x, int ld, int x_off, const float* __restrict__ taps,
                                    const float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ req_of_token, const int* __restrict__ start_pos,
                                    const int* __restrict__ slots, O* __restrict__ out, int out_ld, int C, int K,
                                    int residual, int act) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int r = req_of_token[t];
    const int i = t - cu_seqlens[r];
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float cur[8];
    for (int j = 0; j < K; ++j) {
        const int idx = i - (K - 1) + j;
        float v[8];
        if (idx >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t - (K - 1) + j) * ld + x_off + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        } else if (has_past) {
            const float4* p = reinterpret_cast<const float4*>(state + ((size_t)slot * (K - 1) + (K - 1 + idx)) * C + c);
            const float4 a = p[0], b = p[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        }
        const float4 w0 = *reinterpret_cast<const float4*>(taps + (size_t)j * C + c);
        const float4 w1 = *reinterpret_cast<const float4*>(taps + (size_t)j * C + c + 4);
        acc[0] += w0.x * v[0]; acc[1] += w0.y * v[1]; acc[2] += w0.z * v[2]; acc[3] += w0.w * v[3];
        acc[4] += w1.x * v[4]; acc[5] += w1.y * v[5]; acc[6] += w1.z * v[6]; acc[7] += w1.w * v[7];
        if (j == K - 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) cur[e] = v[e];
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        if (act == 1) acc[e] = acc[e] * sm_sigmoid(acc[e]);
        if (residual) acc[e] += cur[e];
    }
    O* o = out + (size_t)t * out_ld + c;
    if (sizeof(O) == 2) {
        uint4 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        *reinterpret_cast<uint4*>(o) = pk;
    } else {
        reinterpret_cast<float4*>(o)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        reinterpret_cast<float4*>(o)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

// One thread per (request, channel): rows in ascending order, each read from a later row (or from the step's
// tokens) before that row is written.
template <typename A>
__global__ void conv_state_update_kernel(const A* __restrict__ x, int ld, int x_off, float* __restrict__ state,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ start_pos,
                                         const int* __restrict__ slots, int C, int K) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = slots[r];
    if (slot < 0) return;
    const int lo = cu_seqlens[r], n = cu_seqlens[r + 1] - lo;
    if (n <= 0) return;
    const bool has_past = start_pos[r] > 0;
    float* st = state + (size_t)slot * (K - 1) * C + c;
    for (int i = 0; i < K - 1; ++i) {
        const int src = n - (K - 1) + i;
        float v;
        if (src >= 0) v = to_f32(x[(size_t)(lo + src) * ld + x_off + c]);
        else v = has_past ? st[(size_t)(i + n) * C] : 0.f;
        st[(size_t)i * C] = v;
    }
}


extern "C" int rg_causal_conv(const void* x, int x_dtype, int ld, int x_off, const float* taps, const float* state,
                              const int* cu_seqlens, const int* req_of_token, const int* start_pos, const int* slots,
                              void* out, int out_dtype, int out_ld, int T, int C, int K, int residual, int act,
                              void* stream) {
    if (T <= 0 || C <= 0) return 0;
    if (K < 1 || (K > 1 && !state) || act < 0 || act > 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int out_align = out_dtype == RG_DTYPE_BF16 ? 8 : 4;
    if (x_dtype == RG_DTYPE_BF16 && C % 8 == 0 && x_off % 8 == 0 && ld % 8 == 0 && out_ld % out_align == 0 &&
        ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)state & 15) == 0 &&
        ((uintptr_t)taps & 15) == 0) {
        const int th = C / 8 >= 128 ? 128 : 64;
        dim3 g8(T, (C / 8 + th - 1) / th);
        if (g8.y > 65535) return RG_ERR_UNSUPPORTED;
        if (out_dtype == RG_DTYPE_BF16)
            return rg_launch(causal_conv8_kernel<bf16>, g8, dim3(th), 0, s, 1, (const bf16*)x, ld, x_off, taps, state,
                             cu_seqlens, req_of_token, start_pos, slots, (bf16*)out, out_ld, C, K, residual, act);
        if (out_dtype == RG_DTYPE_F32)
            return rg_launch(causal_conv8_kernel<float>, g8, dim3(th), 0, s, 1, (const bf16*)x, ld, x_off, taps, state,
                             cu_seqlens, req_of_token, start_pos, slots, (float*)out, out_ld, C, K, residual, act);
    }
    const int threads = C >= 256 ? 256 : 128;
    dim3 grid(T, (C + threads - 1) / threads);
    if (grid.y > 65535) return RG_ERR_UNSUPPORTED;
#define SM_CONV(A, O) return rg_launch(causal_conv_kernel<A, O>, grid, dim3(threads), 0, s, 1, (const A*)x, ld, x_off, taps, \
        state, cu_seqlens, req_of_token, start_pos, slots, (O*)out, out_ld, C, K, residual, act)
    if (x_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) SM_CONV(bf16, bf16);
    if (x_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_F32) SM_CONV(bf16, float);
    if (x_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) SM_CONV(float, float);
    if (x_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) SM_CONV(float, bf16);
#undef SM_CONV
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_conv_state_update(const void* x, int x_dtype, int ld, int x_off, float* state, const int* cu_seqlens,
                                    const int* start_pos, const int* slots, int R, int C, int K, void* stream) {
    if (R <= 0 || C <= 0 || K <= 1) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = C >= 256 ? 256 : 128;
    dim3 grid(R, (C + threads - 1) / threads);
    if (grid.y > 65535) return RG_ERR_UNSUPPORTED;
    if (x_dtype == RG_DTYPE_BF16)
        return rg_launch(conv_state_update_kernel<bf16>, grid, dim3(threads), 0, s, 1, (const bf16*)x, ld, x_off, state,
                         cu_seqlens, start_pos, slots, C, K);
    if (x_dtype == RG_DTYPE_F32)
        return rg_launch(conv_state_update_kernel<float>, grid, dim3(threads), 0, s, 1, (const float*)x, ld, x_off, state,
                         cu_seqlens, start_pos, slots, C, K);
    return RG_ERR_UNSUPPORTED;
}

// proj rows: [q (H d) | k (H d) | ...] at q_off and k_off.  q_out, k_out [T, H, d] float.  freq: dims / 2 (64-bit).
// act 1: silu on q and k (before the rotation) and, with v_out [T, H dv] float, on the H dv numbers at v_off too.
template <typename A>
__global__ void retention_prepare_kernel(const A* __restrict__ proj, int ld, int q_off, int k_off,
                                         const double* __restrict__ freq, int dims, const int* __restrict__ positions,
                                         float* __restrict__ q_out, float* __restrict__ k_out, int H, int d,
                                         float k_scale, int act, int v_off, int dv, float* __restrict__ v_out) {
    extern __shared__ float cs[];                    // cos | sin of the token's dims / 2 angles
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = dims >> 1;
    const double pos = (double)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) rotary_cos_sin(pos, freq[i], &cs[i], &cs[half + i]);
    __syncthreads();
    const A* row = proj + (size_t)t * ld;
    for (int e = threadIdx.x; e < 2 * H * d; e += blockDim.x) {
        const int which = e / (H * d), rem = e - which * H * d, h = rem / d, i = rem - h * d;
        const A* src = row + (which ? k_off : q_off) + (size_t)h * d;
        float v = to_f32(src[i]);
        if (act) v *= sm_sigmoid(v);
        if (i < dims) {
            float m = to_f32(src[i < half ? i + half : i - half]);
            if (act) m *= sm_sigmoid(m);
            v = i < half ? v * cs[i] - m * cs[half + i] : v * cs[i - half] + m * cs[i];
        }
        if (which) k_out[((size_t)t * H + h) * d + i] = v * k_scale;
        else q_out[((size_t)t * H + h) * d + i] = v;
    }
    if (v_out) {
        for (int e = threadIdx.x; e < H * dv; e += blockDim.x) {
            float v = to_f32(row[v_off + e]);
            if (act) v *= sm_sigmoid(v);
            v_out[(size_t)t * H * dv + e] = v;
        }
    }
}

extern "C" int rg_retention_prepare(const void* proj, int dtype, int ld, int q_off, int k_off, const double* freq,
                                    int dims, const int* positions, float* q_out, float* k_out, int T, int H, int d,
                                    float k_scale, int act, int v_off, int dv, float* v_out, void* stream) {
    if (T <= 0) return 0;
    if (dims < 0 || dims > d || (dims & 1) || H < 1 || d < 1 || act < 0 || act > 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(dims > 0 ? dims : 1) * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    const int threads = 2 * H * d >= 512 ? 256 : 128;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(retention_prepare_kernel<bf16>, dim3(T), dim3(threads), smem, s, 1, (const bf16*)proj, ld, q_off,
                         k_off, freq, dims, positions, q_out, k_out, H, d, k_scale, act, v_off, dv, v_out);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(retention_prepare_kernel<float>, dim3(T), dim3(threads), smem, s, 1, (const float*)proj, ld,
                         q_off, k_off, freq, dims, positions, q_out, k_out, H, d, k_scale, act, v_off, dv, v_out);
    return RG_ERR_UNSUPPORTED;
}

// qk [T, ld] float: q heads (G of d) at column 0, k heads at column G d, in place.  ab: rows ab_ld apart (type A),
// the H numbers b at b_off and the H numbers a at a_off.  beta, g [T, H] float.
template <typename A>
__global__ void delta_prepare_kernel(float* __restrict__ qk, int ld, int G, int d, float q_scale, float unit_eps,
                                     const A* __restrict__ ab, int ab_ld, int b_off, int a_off,
                                     const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                     float* __restrict__ beta, float* __restrict__ g, int H) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* row = qk + (size_t)t * ld;
    for (int hh = warp; hh < 2 * G; hh += nwarp) {
        float* v = row + (size_t)hh * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss + unit_eps) * (hh < G ? q_scale : 1.f);
        for (int i = lane; i < d; i += 32) v[i] *= inv;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float bz = to_f32(ab[(size_t)t * ab_ld + b_off + h]);
        const float az = to_f32(ab[(size_t)t * ab_ld + a_off + h]) + dt_bias[h];
        beta[(size_t)t * H + h] = sm_sigmoid(bz);
        g[(size_t)t * H + h] = expf(-expf(A_log[h]) * sm_softplus(az));
    }
}

extern "C" int rg_delta_prepare(float* qk, int ld, int G, int d, float q_scale, float unit_eps, const void* ab,
                                int ab_dtype, int ab_ld, int b_off, int a_off, const float* A_log, const float* dt_bias,
                                float* beta, float* g, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (G < 1 || d < 1 || H < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 2 * G >= 8 ? 256 : 128;
    if (ab_dtype == RG_DTYPE_BF16)
        return rg_launch(delta_prepare_kernel<bf16>, dim3(T), dim3(threads), 0, s, 1, qk, ld, G, d, q_scale, unit_eps,
                         (const bf16*)ab, ab_ld, b_off, a_off, A_log, dt_bias, beta, g, H);
    if (ab_dtype == RG_DTYPE_F32)
        return rg_launch(delta_prepare_kernel<float>, dim3(T), dim3(threads), 0, s, 1, qk, ld, G, d, q_scale, unit_eps,
                         (const float*)ab, ab_ld, b_off, a_off, A_log, dt_bias, beta, g, H);
    return RG_ERR_UNSUPPORTED;
}

// One block per (request, head, group of CB columns of S).  Thread (j, part) holds DPER rows of column j of S, four
// at a time: rows 4 (i PARTS + part) ... + 3 for i = 0 .. DPER / 4 - 1, so that the PARTS threads of a column, which
// are neighbouring lanes and add their shares with shuffles, read neighbouring 16 bytes of a k or q row (no bank
// conflicts) and of the column's state.  The
// columns of S never meet (S^T k and S^T q are sums down a column), so a head's columns are spread over blocks.
// Tokens are staged in shared memory `chunk` at a time, the next chunk on its way (cp.async for q and k, registers
// for v, g and beta) while this one is worked on; q and k rows are padded with zeros to parts * DPER numbers (rows
// of S beyond d then stay zero without a test in the loop).  q, k: [T, Hqk, d] float rows q_ld / k_ld apart; head h
// reads q/k head h / (H / Hqk).  v: rows v_ld apart (float or bfloat16), head h at column h dv.  decay [H]
// (retention) or g, beta [T, H] (delta rule; beta null: retention).  state [slots, H, dv, d]: S transposed, a
// thread's rows side by side.  o [T, H, dv] float.
//
// The delta rule per token, with a = S_old^T k, b = S_old^T q (one pass over S, reduced together) and c = k . q:
//   u = beta (v - g a);  o = g b + u c;  S <- g S + k u^T
// (c once per token and block, when its chunk has arrived) which is S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with one reduction in the chain from token
// to token instead of two.  Retention: o = decay b + v c;  S <- decay S + k v^T.
#define SCAN_THREADS 128
#define SCAN_MAX_PREFETCH 4       // v numbers of the next chunk a thread holds: chunk * CB <= 4 * threads of the block

__device__ __forceinline__ void scan_cp_async4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void scan_cp_async16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}

template <int DPER, int PARTS, bool DELTA, typename V>
__global__ void __launch_bounds__(SCAN_THREADS)
state_scan_kernel(const float* __restrict__ q, int q_ld, const float* __restrict__ k, int k_ld,
                  const V* __restrict__ v, int v_ld, const float* __restrict__ decay,
                  const float* __restrict__ g, const float* __restrict__ beta,
                  float* __restrict__ state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ start_pos, const int* __restrict__ slots,
                  float* __restrict__ o, int H, int Hqk, int d, int dv, int CB, int chunk, int vec) {
    extern __shared__ __align__(16) float sm[];
    constexpr int parts = PARTS;
    constexpr int DP = PARTS * DPER;                 // padded length of a q or k row
    const int stage = chunk * (2 * DP + CB + 4);     // floats of one stage: q, k [chunk][DP], v [chunk][CB], (g, beta, c, -) [chunk]
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * CB;
    const int hq = h / (H / Hqk);
    const int lo = cu_seqlens[r], hi = cu_seqlens[r + 1];
    if (hi <= lo) return;
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    const int jl = threadIdx.x / parts, part = threadIdx.x - jl * parts;
    const int j = j0 + jl;
    const bool live = jl < CB && j < dv;
    float* st = (slot >= 0 && live) ? state + (((size_t)slot * H + h) * dv + j) * d : nullptr;   // the column's d numbers
    float S[DPER];
#pragma unroll
    for (int i4 = 0; i4 < DPER / 4; ++i4) {
        const int r0 = 4 * (i4 * PARTS + part);
        if (st && has_past && vec && r0 < d) {
            const float4 x = *reinterpret_cast<const float4*>(st + r0);
            S[4 * i4] = x.x; S[4 * i4 + 1] = x.y; S[4 * i4 + 2] = x.z; S[4 * i4 + 3] = x.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) S[4 * i4 + i] = (st && has_past && r0 + i < d) ? st[r0 + i] : 0.f;
        }
    }
    const float fixed = decay ? decay[h] : 1.f;
    const int ncols = min(CB, dv - j0);
    // the padding of q and k rows is zero in both stages, once
    if (DP > d) {
        for (int e = threadIdx.x; e < 2 * chunk * (DP - d); e += blockDim.x) {
            const int stg = e / (chunk * (DP - d)), rem = e - stg * chunk * (DP - d);
            const int tt = rem / (DP - d), i = d + rem - tt * (DP - d);
            sm[stg * stage + tt * DP + i] = 0.f;
            sm[stg * stage + chunk * DP + tt * DP + i] = 0.f;
        }
    }
    float pv[SCAN_MAX_PREFETCH], pg = 0.f, pb = 0.f;
    // this thread's places in a chunk's tile of v (the same in every chunk), and in the rows of q and k
    int v_tt[SCAN_MAX_PREFETCH], v_i[SCAN_MAX_PREFETCH];
#pragma unroll
    for (int x = 0; x < SCAN_MAX_PREFETCH; ++x) {
        const int e = threadIdx.x + x * blockDim.x;
        v_tt[x] = e < chunk * ncols ? e / ncols : chunk;
        v_i[x] = e - v_tt[x] * ncols;
    }
    const V* vh = v + (size_t)h * dv + j0;
    const float* qh = q + (size_t)hq * d;
    const float* kh = k + (size_t)hq * d;
    const int d4 = d >> 2;
    const bool by_rows = vec && d4 <= (int)blockDim.x;               // whole rows per pass: no division in the loop
    const int rpp = by_rows ? blockDim.x / d4 : 1, row_t = threadIdx.x / (by_rows ? d4 : 1),
              row_i = by_rows ? (threadIdx.x - row_t * d4) * 4 : 0;
    // q and k of `n` tokens from `base` on into stage `stg`, asynchronously
    auto issue = [&](int stg, int base, int n) {
        float* sq = sm + stg * stage;
        float* sk = sq + chunk * DP;
        if (by_rows) {
            if (row_t < rpp)
                for (int tt = row_t; tt < n; tt += rpp) {
                    scan_cp_async16(sq + tt * DP + row_i, qh + (size_t)(base + tt) * q_ld + row_i);
                    scan_cp_async16(sk + tt * DP + row_i, kh + (size_t)(base + tt) * k_ld + row_i);
                }
        } else if (vec) {
            for (int e = threadIdx.x; e < n * d4; e += blockDim.x) {
                const int tt = e / d4, i = (e - tt * d4) * 4;
                scan_cp_async16(sq + tt * DP + i, q + (size_t)(base + tt) * q_ld + (size_t)hq * d + i);
                scan_cp_async16(sk + tt * DP + i, k + (size_t)(base + tt) * k_ld + (size_t)hq * d + i);
            }
        } else {
            for (int e = threadIdx.x; e < n * d; e += blockDim.x) {
                const int tt = e / d, i = e - tt * d;
                scan_cp_async4(sq + tt * DP + i, q + (size_t)(base + tt) * q_ld + (size_t)hq * d + i);
                scan_cp_async4(sk + tt * DP + i, k + (size_t)(base + tt) * k_ld + (size_t)hq * d + i);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // v, g and beta of those tokens into registers; `park` leaves them in the stage
    auto fetch = [&](int base, int n) {
#pragma unroll
        for (int x = 0; x < SCAN_MAX_PREFETCH; ++x)
            if (v_tt[x] < n) pv[x] = to_f32(vh[(size_t)(base + v_tt[x]) * v_ld + v_i[x]]);
        if ((int)threadIdx.x < n) {
            pg = g ? g[(size_t)(base + threadIdx.x) * H + h] : fixed;
            pb = beta ? beta[(size_t)(base + threadIdx.x) * H + h] : 0.f;
        }
    };
    auto park = [&](int stg, int n) {
        float* sv = sm + stg * stage + 2 * chunk * DP;
#pragma unroll
        for (int x = 0; x < SCAN_MAX_PREFETCH; ++x)
            if (v_tt[x] < n) sv[v_tt[x] * CB + v_i[x]] = pv[x];
        if ((int)threadIdx.x < n) {
            sv[chunk * CB + 4 * threadIdx.x] = pg;
            sv[chunk * CB + 4 * threadIdx.x + 1] = pb;
        }
    };
    float* op = o + ((size_t)lo * H + h) * dv + (live ? j : 0);
    const size_t ostep = (size_t)H * dv;
    issue(0, lo, min(chunk, hi - lo));
    fetch(lo, min(chunk, hi - lo));
    int stg = 0;
    for (int base = lo; base < hi; base += chunk, stg ^= 1) {
        const int n = min(chunk, hi - base);
        park(stg, n);
        const int nb = base + chunk;
        __syncthreads();                                            // the other stage's readers are done
        if (nb < hi) {
            issue(stg ^ 1, nb, min(chunk, hi - nb));
            fetch(nb, min(chunk, hi - nb));
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();                                            // this stage is complete for everybody
        const float* sq = sm + stg * stage;
        const float* sk = sq + chunk * DP;
        const float* sv = sk + chunk * DP;
        float* sgbc = sm + stg * stage + chunk * (2 * DP + CB);      // (g, beta, c, -) of every token
        // c = k . q of the chunk's tokens, eight lanes a token
        // (every lane runs every round of the loop, so that the shuffles meet whole warps)
        for (int t0 = 0; t0 < n; t0 += blockDim.x >> 3) {
            const int tt = t0 + (threadIdx.x >> 3);
            float c = 0.f;
            if (tt < n) {
                const float4* k4 = reinterpret_cast<const float4*>(sk + tt * DP);
                const float4* q4 = reinterpret_cast<const float4*>(sq + tt * DP);
                for (int i = threadIdx.x & 7; i < DP / 4; i += 8) {
                    const float4 a = k4[i], b = q4[i];
                    c += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
                }
            }
            c += __shfl_xor_sync(0xffffffffu, c, 1);
            c += __shfl_xor_sync(0xffffffffu, c, 2);
            c += __shfl_xor_sync(0xffffffffu, c, 4);
            if (tt < n && (threadIdx.x & 7) == 0) sgbc[4 * tt + 2] = c;
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < n; ++tt) {
            const float4* kt = reinterpret_cast<const float4*>(sk + tt * DP) + part;
            const float4* qt = reinterpret_cast<const float4*>(sq + tt * DP) + part;
            const float4 gbc = *reinterpret_cast<const float4*>(sgbc + 4 * tt);
            const float gt = gbc.x;
            float kk[DPER];
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int i4 = 0; i4 < DPER / 4; ++i4) {
                const float4 k4 = kt[i4 * PARTS], q4 = qt[i4 * PARTS];
                kk[4 * i4] = k4.x; kk[4 * i4 + 1] = k4.y; kk[4 * i4 + 2] = k4.z; kk[4 * i4 + 3] = k4.w;
                if (DELTA) {
                    a0 += S[4 * i4] * k4.x;     a1 += S[4 * i4 + 1] * k4.y;
                    a0 += S[4 * i4 + 2] * k4.z; a1 += S[4 * i4 + 3] * k4.w;
                }
                b0 += S[4 * i4] * q4.x;     b1 += S[4 * i4 + 1] * q4.y;
                b0 += S[4 * i4 + 2] * q4.z; b1 += S[4 * i4 + 3] * q4.w;
            }
            float a = a0 + a1, b = b0 + b1;
            const float c = gbc.z;
#pragma unroll
            for (int off = PARTS >> 1; off > 0; off >>= 1) {
                if (DELTA) a += __shfl_xor_sync(0xffffffffu, a, off);
                b += __shfl_xor_sync(0xffffffffu, b, off);
            }
            float u = live ? sv[tt * CB + jl] : 0.f;
            if (DELTA) u = gbc.y * (u - gt * a);
#pragma unroll
            for (int i = 0; i < DPER; ++i) S[i] = S[i] * gt + kk[i] * u;
            if (live && part == 0) *op = gt * b + u * c;
            op += ostep;
        }
    }
    if (st) {
#pragma unroll
        for (int i4 = 0; i4 < DPER / 4; ++i4) {
            const int r0 = 4 * (i4 * PARTS + part);
            if (vec && r0 < d) {
                *reinterpret_cast<float4*>(st + r0) = make_float4(S[4 * i4], S[4 * i4 + 1], S[4 * i4 + 2], S[4 * i4 + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (r0 + i < d) st[r0 + i] = S[4 * i4 + i];
            }
        }
    }
}

// For measurements: rows of S per thread (4, 8, 16 or 32) instead of the launcher's own choice; 0 gives it back.
static int rg_scan_rows_override = 0;
extern "C" void rg_state_scan_rows(int rows) { rg_scan_rows_override = rows; }

extern "C" int rg_state_scan(const float* q, int q_ld, const float* k, int k_ld, const void* v, int v_dtype, int v_ld,
                             const float* decay, const float* g, const float* beta, float* state,
                             const int* cu_seqlens, const int* start_pos, const int* slots, float* o, int R, int H,
                             int Hqk, int d, int dv, void* stream) {
    if (R <= 0) return 0;
    if (H < 1 || Hqk < 1 || H % Hqk || d < 1 || dv < 1 || d > 256 || (!decay && !g) || (beta && !g))
        return RG_ERR_UNSUPPORTED;
    // Rows of S per thread: 8 up to d = 64, then 16, then 32; `parts` (a power of two) threads share a column, and a
    // block of at most SCAN_THREADS threads takes CB columns.  While that gives fewer blocks than SMs (a long prompt
    // alone), threads take half as many rows each, down to 8 (measured, one prompt of 4,096 tokens, 16 heads of
    // 128 x 128, with 16 / 8 / 4 rows: retention 1.04 / 0.98 / 0.90 ms, the delta rule 0.97 / 1.05 / 1.35 ms; with
    // 4 rows the delta rule's reduction over 32 lanes lies on the path from token to token).
    int dper = d <= 64 ? 8 : (d <= 128 ? 16 : 32);
    auto shape = [&](int dp, int& parts, int& CB, int& col_blocks) {
        parts = 1;
        while (parts * dp < d) parts <<= 1;
        CB = SCAN_THREADS / parts;
        if (CB > dv) CB = dv;
        col_blocks = (dv + CB - 1) / CB;
    };
    int parts, CB, col_blocks;
    shape(dper, parts, CB, col_blocks);
    if (rg_scan_rows_override > 0) {
        dper = rg_scan_rows_override;
        shape(dper, parts, CB, col_blocks);
        if (parts > 32 || parts * dper > 256) return RG_ERR_UNSUPPORTED;
    } else
    while ((long long)R * H * col_blocks < 148 && dper > 8) {
        int p2, c2, b2;
        shape(dper / 2, p2, c2, b2);
        if (p2 > 32) break;
        dper /= 2; parts = p2; CB = c2; col_blocks = b2;
    }
    const int threads = ((parts * CB + 31) / 32) * 32;
    const int DP = parts * dper;
    int chunk = DP > 128 ? 8 : 16;
    if (chunk > 4 * parts) chunk = 4 * parts;                      // what a thread prefetches of v stays in 4 registers
    if (chunk * CB > SCAN_MAX_PREFETCH * threads) return RG_ERR_UNSUPPORTED;
    const size_t smem = (size_t)2 * chunk * (2 * DP + CB + 4) * sizeof(float);
    if (smem > 48 * 1024 || H > 65535 || col_blocks > 65535) return RG_ERR_UNSUPPORTED;
    // 16-byte copies and state accesses where every row starts on a 16-byte boundary
    const int vec = d % 4 == 0 && q_ld % 4 == 0 && k_ld % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 &&
                    ((uintptr_t)state & 15) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(R, H, col_blocks);
#define SM_SCAN(DP_, PA_, DE_, V) return rg_launch(state_scan_kernel<DP_, PA_, DE_, V>, grid, dim3(threads), smem, s, 1, \
        q, q_ld, k, k_ld, (const V*)v, v_ld, decay, g, beta, state, cu_seqlens, start_pos, slots, o, H, Hqk, d, dv, CB, \
        chunk, vec)
#define SM_SCAN_RULE(DP_, PA_, V) { if (beta) SM_SCAN(DP_, PA_, true, V); SM_SCAN(DP_, PA_, false, V); }
#define SM_SCAN_PARTS(DP_, V) switch (parts) { \
        case 1: SM_SCAN_RULE(DP_, 1, V) case 2: SM_SCAN_RULE(DP_, 2, V) case 4: SM_SCAN_RULE(DP_, 4, V) \
        case 8: SM_SCAN_RULE(DP_, 8, V) case 16: if (DP_ <= 16) SM_SCAN_RULE(DP_ <= 16 ? DP_ : 16, 16, V) break; \
        case 32: if (DP_ <= 8) SM_SCAN_RULE(DP_ <= 8 ? DP_ : 8, 32, V) break; default: break; } \
        return RG_ERR_UNSUPPORTED;
#define SM_SCAN_ROWS(V) switch (dper) { case 4: SM_SCAN_PARTS(4, V) case 8: SM_SCAN_PARTS(8, V) \
        case 16: SM_SCAN_PARTS(16, V) case 32: SM_SCAN_PARTS(32, V) default: return RG_ERR_UNSUPPORTED; }
    if (v_dtype == RG_DTYPE_F32) SM_SCAN_ROWS(float)
    if (v_dtype == RG_DTYPE_BF16) SM_SCAN_ROWS(bf16)
    return RG_ERR_UNSUPPORTED;
#undef SM_SCAN_ROWS
#undef SM_SCAN_PARTS
#undef SM_SCAN_RULE
#undef SM_SCAN
}

// o [T, H, dv] float; gate: rows gate_ld apart (type A), head h at column gate_off + h dv; weight [dv] or null.
// out [T, H dv] (type A) = o / sqrt(mean(o^2) + eps) * weight * silu(gate) (gate_kind 1: sigmoid(gate)).  One warp
// per (token, head).
template <typename A, typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const A* __restrict__ gate, int gate_ld, int gate_off,
                                      const float* __restrict__ weight, float eps, O* __restrict__ out, int T, int H,
                                      int dv, int gate_kind) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= (long long)T * H) return;
    const int t = (int)(idx / H), h = (int)(idx - (long long)t * H);
    const float* src = o + (size_t)idx * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += src[i] * src[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps);
    const A* grow = gate + (size_t)t * gate_ld + gate_off + (size_t)h * dv;
    for (int i = lane; i < dv; i += 32) {
        const float z = to_f32(grow[i]);
        out[(size_t)idx * dv + i] = from_f32<O>(src[i] * inv * (weight ? weight[i] : 1.f) *
                                                (gate_kind ? sm_sigmoid(z) : z * sm_sigmoid(z)));
    }
}

// The same with ONE root mean square over all H dv numbers of a token and a weight of that size: one block per token.
template <typename A, typename O>
__global__ void row_norm_gate_kernel(const float* __restrict__ o, const A* __restrict__ gate, int gate_ld, int gate_off,
                                     const float* __restrict__ weight, float eps, O* __restrict__ out, int n,
                                     int gate_kind) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const float* src = o + (size_t)t * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += src[i] * src[i];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)n + eps);
    const A* grow = gate + (size_t)t * gate_ld + gate_off;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float z = to_f32(grow[i]);
        out[(size_t)t * n + i] = from_f32<O>(src[i] * inv * (weight ? weight[i] : 1.f) *
                                             (gate_kind ? sm_sigmoid(z) : z * sm_sigmoid(z)));
    }
}

// whole 0: every head normed on its own (weight [dv]); 1: all heads of a token together (weight [H dv]).
// gate_kind 0: silu(gate); 1: sigmoid(gate).
extern "C" int rg_head_norm_gate(const float* o, const void* gate, int gate_dtype, int gate_ld, int gate_off,
                                 const float* weight, float eps, void* out, int out_dtype, int T, int H, int dv,
                                 int whole, int gate_kind, void* stream) {
    if (T <= 0) return 0;
    if (gate_kind < 0 || gate_kind > 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const long long n = (long long)T * H;
    dim3 grid((unsigned)((n + 3) / 4));
    const int row = H * dv;
    const int threads = row >= 1024 ? 256 : 128;
#define SM_HNG(A, O) { if (whole) return rg_launch(row_norm_gate_kernel<A, O>, dim3(T), dim3(threads), 0, s, 1, o, \
        (const A*)gate, gate_ld, gate_off, weight, eps, (O*)out, row, gate_kind); \
        return rg_launch(head_norm_gate_kernel<A, O>, grid, dim3(128), 0, s, 1, o, (const A*)gate, gate_ld, \
        gate_off, weight, eps, (O*)out, T, H, dv, gate_kind); }
    if (gate_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) SM_HNG(bf16, bf16)
    if (gate_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) SM_HNG(float, float)
    if (gate_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) SM_HNG(float, bf16)
#undef SM_HNG
    return RG_ERR_UNSUPPORTED;
}
