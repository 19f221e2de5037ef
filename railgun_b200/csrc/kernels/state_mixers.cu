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

// x: rows ld apart, channel c at column x_off + c.  state [slots, K - 1, C] float, oldest input first.
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
        acc += taps[(size_t)c * K + j] * v;
    }
    if (act == 1) acc = acc * sm_sigmoid(acc);
    if (residual) acc += to_f32(x[(size_t)t * ld + x_off + c]);
    out[(size_t)t * out_ld + c] = from_f32<O>(acc);
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
template <typename A>
__global__ void retention_prepare_kernel(const A* __restrict__ proj, int ld, int q_off, int k_off,
                                         const double* __restrict__ freq, int dims, const int* __restrict__ positions,
                                         float* __restrict__ q_out, float* __restrict__ k_out, int H, int d,
                                         float k_scale) {
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
        if (i < half) v = v * cs[i] - to_f32(src[i + half]) * cs[half + i];
        else if (i < dims) v = v * cs[i - half] + to_f32(src[i - half]) * cs[i];
        if (which) k_out[((size_t)t * H + h) * d + i] = v * k_scale;
        else q_out[((size_t)t * H + h) * d + i] = v;
    }
}

extern "C" int rg_retention_prepare(const void* proj, int dtype, int ld, int q_off, int k_off, const double* freq,
                                    int dims, const int* positions, float* q_out, float* k_out, int T, int H, int d,
                                    float k_scale, void* stream) {
    if (T <= 0) return 0;
    if (dims < 0 || dims > d || (dims & 1) || H < 1 || d < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(dims > 0 ? dims : 1) * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    const int threads = 2 * H * d >= 512 ? 256 : 128;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(retention_prepare_kernel<bf16>, dim3(T), dim3(threads), smem, s, 1, (const bf16*)proj, ld, q_off,
                         k_off, freq, dims, positions, q_out, k_out, H, d, k_scale);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(retention_prepare_kernel<float>, dim3(T), dim3(threads), smem, s, 1, (const float*)proj, ld,
                         q_off, k_off, freq, dims, positions, q_out, k_out, H, d, k_scale);
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

// One block per (request, head).  Thread (j, part) holds DPER rows of column j of S: rows part * DPER ...; the
// `parts` threads of a column are neighbouring lanes and add their shares with shuffles.  Tokens are staged in
// shared memory SCAN_CHUNK at a time.  q, k: [T, Hqk, d] float rows q_ld / k_ld apart; head h reads q/k head
// h / (H / Hqk).  v: rows v_ld apart (float or bfloat16), head h at column h dv.  decay [H] (retention) or g, beta [T, H]
// (delta rule; beta null: retention).  state [slots, H, d, dv].  o [T, H, dv] float.
#define SCAN_CHUNK 16
template <int DPER, typename V>
__global__ void state_scan_kernel(const float* __restrict__ q, int q_ld, const float* __restrict__ k, int k_ld,
                                  const V* __restrict__ v, int v_ld, const float* __restrict__ decay,
                                  const float* __restrict__ g, const float* __restrict__ beta,
                                  float* __restrict__ state, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ start_pos, const int* __restrict__ slots,
                                  float* __restrict__ o, int H, int Hqk, int d, int dv, int parts) {
    extern __shared__ float sm[];
    float* sq = sm;                                  // [CHUNK][d]
    float* sk = sq + SCAN_CHUNK * d;                 // [CHUNK][d]
    float* sv = sk + SCAN_CHUNK * d;                 // [CHUNK][dv]
    float* sg = sv + SCAN_CHUNK * dv;                // [CHUNK]
    float* sb = sg + SCAN_CHUNK;                     // [CHUNK]
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y;
    const int hq = h / (H / Hqk);
    const int lo = cu_seqlens[r], hi = cu_seqlens[r + 1];
    if (hi <= lo) return;
    const int slot = slots[r];
    const bool has_past = slot >= 0 && start_pos[r] > 0;
    const int j = threadIdx.x / parts, part = threadIdx.x - j * parts;
    const bool live = j < dv;
    const int d0 = part * DPER;
    float* st = slot >= 0 ? state + ((size_t)slot * H + h) * d * dv : nullptr;
    float S[DPER];
#pragma unroll
    for (int i = 0; i < DPER; ++i)
        S[i] = (has_past && live && d0 + i < d) ? st[(size_t)(d0 + i) * dv + j] : 0.f;
    const float fixed = decay ? decay[h] : 1.f;
    for (int base = lo; base < hi; base += SCAN_CHUNK) {
        const int n = min(SCAN_CHUNK, hi - base);
        __syncthreads();
        for (int e = threadIdx.x; e < n * d; e += blockDim.x) {
            const int tt = e / d, i = e - tt * d;
            sq[e] = q[(size_t)(base + tt) * q_ld + (size_t)hq * d + i];
            sk[e] = k[(size_t)(base + tt) * k_ld + (size_t)hq * d + i];
        }
        for (int e = threadIdx.x; e < n * dv; e += blockDim.x) {
            const int tt = e / dv, i = e - tt * dv;
            sv[e] = to_f32(v[(size_t)(base + tt) * v_ld + (size_t)h * dv + i]);
        }
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            sg[e] = g ? g[(size_t)(base + e) * H + h] : fixed;
            sb[e] = beta ? beta[(size_t)(base + e) * H + h] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float* kt = sk + tt * d + d0;
            const float* qt = sq + tt * d + d0;
            const float gt = sg[tt];
            float u = live ? sv[tt * dv + j] : 0.f;
            if (beta) {
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < DPER; ++i) {
                    S[i] *= gt;
                    if (d0 + i < d) dot += S[i] * kt[i];
                }
                for (int off = parts >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
                u = sb[tt] * (u - dot);
            } else {
#pragma unroll
                for (int i = 0; i < DPER; ++i) S[i] *= gt;
            }
            float out = 0.f;
#pragma unroll
            for (int i = 0; i < DPER; ++i) {
                if (d0 + i < d) {
                    S[i] += kt[i] * u;
                    out += S[i] * qt[i];
                }
            }
            for (int off = parts >> 1; off > 0; off >>= 1) out += __shfl_xor_sync(0xffffffffu, out, off);
            if (live && part == 0) o[((size_t)(base + tt) * H + h) * dv + j] = out;
        }
    }
    if (st && live) {
#pragma unroll
        for (int i = 0; i < DPER; ++i)
            if (d0 + i < d) st[(size_t)(d0 + i) * dv + j] = S[i];
    }
}

extern "C" int rg_state_scan(const float* q, int q_ld, const float* k, int k_ld, const void* v, int v_dtype, int v_ld,
                             const float* decay, const float* g, const float* beta, float* state,
                             const int* cu_seqlens, const int* start_pos, const int* slots, float* o, int R, int H,
                             int Hqk, int d, int dv, void* stream) {
    if (R <= 0) return 0;
    if (H < 1 || Hqk < 1 || H % Hqk || d < 1 || dv < 1 || d > 256 || dv > 1024 || (!decay && !g) || (beta && !g))
        return RG_ERR_UNSUPPORTED;
    // rows of S per thread: 8 up to d = 64, then 16, then 32 (`parts` a power of two, at most 32 lanes wide;
    // parts * columns at most 1024 threads)
    int dper = d <= 64 ? 8 : (d <= 128 ? 16 : 32);
    int parts = 1;
    while (parts * dper < d) parts <<= 1;
    while (parts > 1 && (long long)parts * dv > 1024) { parts >>= 1; dper <<= 1; }
    if (dper > 32 || parts > 32) return RG_ERR_UNSUPPORTED;
    int threads = ((parts * dv + 31) / 32) * 32;
    if (threads > 1024) return RG_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(SCAN_CHUNK * (2 * d + dv) + 2 * SCAN_CHUNK) * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    if (H > 65535) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(R, H);
#define SM_SCAN(DP, V) return rg_launch(state_scan_kernel<DP, V>, grid, dim3(threads), smem, s, 1, q, q_ld, k, k_ld, \
        (const V*)v, v_ld, decay, g, beta, state, cu_seqlens, start_pos, slots, o, H, Hqk, d, dv, parts)
    if (v_dtype == RG_DTYPE_F32) {
        if (dper == 8) SM_SCAN(8, float);
        if (dper == 16) SM_SCAN(16, float);
        SM_SCAN(32, float);
    }
    if (v_dtype == RG_DTYPE_BF16) {
        if (dper == 8) SM_SCAN(8, bf16);
        if (dper == 16) SM_SCAN(16, bf16);
        SM_SCAN(32, bf16);
    }
    return RG_ERR_UNSUPPORTED;
#undef SM_SCAN
}

// o [T, H, dv] float; gate: rows gate_ld apart (type A), head h at column gate_off + h dv; weight [dv] or null.
// out [T, H dv] (type A) = o / sqrt(mean(o^2) + eps) * weight * silu(gate).  One warp per (token, head).
template <typename A, typename O>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const A* __restrict__ gate, int gate_ld, int gate_off,
                                      const float* __restrict__ weight, float eps, O* __restrict__ out, int T, int H,
                                      int dv) {
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
        out[(size_t)idx * dv + i] = from_f32<O>(src[i] * inv * (weight ? weight[i] : 1.f) * (z * sm_sigmoid(z)));
    }
}

extern "C" int rg_head_norm_gate(const float* o, const void* gate, int gate_dtype, int gate_ld, int gate_off,
                                 const float* weight, float eps, void* out, int out_dtype, int T, int H, int dv,
                                 void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long n = (long long)T * H;
    dim3 grid((unsigned)((n + 3) / 4));
#define SM_HNG(A, O) return rg_launch(head_norm_gate_kernel<A, O>, grid, dim3(128), 0, s, 1, o, (const A*)gate, gate_ld, \
        gate_off, weight, eps, (O*)out, T, H, dv)
    if (gate_dtype == RG_DTYPE_BF16 && out_dtype == RG_DTYPE_BF16) SM_HNG(bf16, bf16);
    if (gate_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_F32) SM_HNG(float, float);
    if (gate_dtype == RG_DTYPE_F32 && out_dtype == RG_DTYPE_BF16) SM_HNG(float, bf16);
#undef SM_HNG
    return RG_ERR_UNSUPPORTED;
}
