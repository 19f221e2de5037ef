// Routed experts: the router, the grouping of (token, choice) pairs by expert, the experts' products over
// those groups, and the weighted sum.
//
//   z = W_r h (32-bit), s = softmax(z) over all N router outputs (or, scoring 1, s = sigmoid(z), each on its own)
//   the `top` outputs with the largest s + correction are chosen; their weights are s / (sum of the chosen s
//   + 1e-20).  Outputs E..N-1 stand for identity experts (the expert's result is h itself); outputs 0..E-1
//   for gated experts  down(silu(gate h) * (up h)).
//   out = sum_k weight_k * expert_k(h)  (+ an always-on shared expert's result, computed elsewhere)
//
// Nothing here is planned on the host: the number of rows every expert gets is only known on the device, so
// the products run over a list of row tiles that `moe_align` writes (at most pairs / tile + E of them; the
// launch covers that bound and unused tiles return at once), which keeps a step capturable in a CUDA graph.
//
//   moe_route          one block per four tokens: its warps (up to 32) share the router's rows, then take a token each
//   moe_align          one block: counts per expert, segment starts, the pairs in expert order, the tile list
//   moe_grouped_gemm   32-bit arithmetic on CUDA cores, any sizes and both storage types (the true 32-bit path)
//   moe_combine        one block per token, 32-bit sum in the order of the choices
#include "common.cuh"

#define ROUTE_TOKENS 4        // tokens per block: a router row is read once for all of them

template <typename A>
__global__ void moe_route_kernel(const A* __restrict__ x, const float* __restrict__ router,
                                 const float* __restrict__ correction, int* __restrict__ ids,
                                 float* __restrict__ weights, int T, int W, int N, int top, int renormalize,
                                 int scoring) {
    extern __shared__ float sm[];                 // per token of the block: N scores, N choice scores
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int t0 = blockIdx.x * ROUTE_TOKENS;
    const int nt = min(ROUTE_TOKENS, T - t0);
    float* base = sm;
    // every lane adds its own elements in index order (four at a time where rows start on 16-byte boundaries),
    // then the lanes are added up: a token's logits do not depend on what else is in the step
    const bool vec = (W & 3) == 0 && sizeof(A) == 2;
    for (int n = warp; n < N; n += nwarps) {
        const float* wr = router + (size_t)n * W;
        float dot[ROUTE_TOKENS];
#pragma unroll
        for (int j = 0; j < ROUTE_TOKENS; ++j) dot[j] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int i = lane * 4; i < W; i += 128) {
                const float4 r = *reinterpret_cast<const float4*>(wr + i);
#pragma unroll
                for (int j = 0; j < ROUTE_TOKENS; ++j) {
                    if (j < nt) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)(t0 + j) * W + i);
                        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                        dot[j] += r.x * __low2float(lo);
                        dot[j] += r.y * __high2float(lo);
                        dot[j] += r.z * __low2float(hi);
                        dot[j] += r.w * __high2float(hi);
                    }
                }
            }
        } else {
            for (int i = lane; i < W; i += 32) {
                const float r = wr[i];
#pragma unroll
                for (int j = 0; j < ROUTE_TOKENS; ++j)
                    if (j < nt) dot[j] += r * to_f32(x[(size_t)(t0 + j) * W + i]);
            }
        }
#pragma unroll
        for (int j = 0; j < ROUTE_TOKENS; ++j) {
            const float d = warp_sum(dot[j]);
            if (lane == 0) base[(size_t)j * 2 * N + n] = d;
        }
    }
    __syncthreads();
    for (int j = warp; j < nt; j += nwarps) {
        const int t = t0 + j;
        float* s = base + (size_t)j * 2 * N;
        float* c = s + N;
        if (scoring == 1) {
            // without a correction the largest scores are the largest logits, which do not saturate
            for (int n = lane; n < N; n += 32) {
                const float z = s[n];
                const float p = 1.f / (1.f + expf(-z));
                s[n] = p;
                c[n] = correction ? p + correction[n] : z;
            }
        } else {
            float mx = -INFINITY;
            for (int n = lane; n < N; n += 32) mx = fmaxf(mx, s[n]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int n = lane; n < N; n += 32) { const float e = expf(s[n] - mx); s[n] = e; sum += e; }
            sum = warp_sum(sum);
            const float inv = 1.f / sum;
            for (int n = lane; n < N; n += 32) { const float p = s[n] * inv; s[n] = p; c[n] = p + (correction ? correction[n] : 0.f); }
        }
        __syncwarp();
        float chosen_sum = 0.f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int arg = N;
            for (int n = lane; n < N; n += 32)
                if (c[n] > best) { best = c[n]; arg = n; }         // the lowest index among a lane's equals
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg >= N) arg = 0;                                  // only if every score is NaN or -inf
            const float p = s[arg];
            chosen_sum += p;
            if (lane == 0) {
                ids[(size_t)t * top + k] = arg;
                weights[(size_t)t * top + k] = p;
                c[arg] = -INFINITY;
            }
            __syncwarp();
        }
        const float norm = renormalize ? 1.f / (chosen_sum + 1e-20f) : 1.f;
        for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= norm;
        __syncwarp();
    }
}

extern "C" int rg_moe_route(const void* x, int dtype, const float* router, const float* correction, int* ids,
                            float* weights, int T, int W, int N, int top, int renormalize, int scoring, void* stream) {
    if (T <= 0) return 0;
    if (top < 1 || top > N || scoring < 0 || scoring > 1) return RG_ERR_UNSUPPORTED;
    const size_t smem = (size_t)ROUTE_TOKENS * 2 * N * sizeof(float);
    if (smem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = N < 4 ? 4 : (N > 32 ? 32 : N);               // a warp per router row, up to 32
    dim3 grid((T + ROUTE_TOKENS - 1) / ROUTE_TOKENS), block(warps * 32);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(moe_route_kernel<bf16>, grid, block, smem, s, 1, (const bf16*)x, router, correction, ids,
                         weights, T, W, N, top, renormalize, scoring);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(moe_route_kernel<float>, grid, block, smem, s, 1, (const float*)x, router, correction, ids,
                         weights, T, W, N, top, renormalize, scoring);
    return RG_ERR_UNSUPPORTED;
}

// ids: [P] chosen router outputs of the P = T * top pairs.  Pairs whose output is >= E (identity experts) get
// no place.  sorted_pair[pos] = pair at place pos (-1 for the places left over); pair_pos[pair] = its place or -1; tiles[i] = (expert, first
// place, places) in tiles of `tile_rows`, expert -1 for the unused tail of the list (max_tiles entries).
__global__ void moe_align_kernel(const int* __restrict__ ids, int P, int E, int tile_rows, int* __restrict__ sorted_pair,
                                 int* __restrict__ pair_pos, int* __restrict__ tiles, int max_tiles) {
    extern __shared__ int ism[];                  // count[E], start[E + 1], fill[E], tile_start[E + 1]
    int* count = ism;
    int* start = count + E;
    int* fill = start + E + 1;
    int* tstart = fill + E;
    pdl_wait();
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0, b = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = a;
            tstart[e] = b;
            a += count[e];
            b += (count[e] + tile_rows - 1) / tile_rows;
        }
        start[E] = a;
        tstart[E] = b;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = -1;
        if (e >= 0 && e < E) {
            pos = start[e] + atomicAdd(&fill[e], 1);
            sorted_pair[pos] = p;
        }
        pair_pos[p] = pos;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = tstart[e + 1] - tstart[e];
        for (int i = 0; i < n; ++i) {
            int* tl = tiles + 3 * (size_t)(tstart[e] + i);
            tl[0] = e;
            tl[1] = start[e] + i * tile_rows;
            tl[2] = min(tile_rows, count[e] - i * tile_rows);
        }
    }
    for (int pos = start[E] + threadIdx.x; pos < P; pos += blockDim.x) sorted_pair[pos] = -1;   // places nobody has
    for (int i = tstart[E] + threadIdx.x; i < max_tiles; i += blockDim.x) {
        tiles[3 * (size_t)i] = -1;
        tiles[3 * (size_t)i + 1] = 0;
        tiles[3 * (size_t)i + 2] = 0;
    }
}

extern "C" int rg_moe_align(const int* ids, int P, int E, int tile_rows, int* sorted_pair, int* pair_pos, int* tiles,
                            int max_tiles, void* stream) {
    if (P <= 0) return 0;
    const size_t smem = (size_t)(4 * E + 2) * sizeof(int);
    if (E < 1 || smem > 48 * 1024 || tile_rows < 1 || max_tiles < (P + tile_rows - 1) / tile_rows + E)
        return RG_ERR_UNSUPPORTED;
    return rg_launch(moe_align_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, 1, ids, P, E, tile_rows,
                     sorted_pair, pair_pos, tiles, max_tiles);
}

// One tile of the list: rows [first, first + n) of expert e.  Row `pos` of A is a[src[pos] / src_div] when
// src is given (the token of the pair at that place), else a[pos].  w: [E, (GATED ? 2 N : N), K], the gated
// form holding N gate rows and then N up rows per expert; out[pos, n] = sum_k a_k w_nk, or with GATED
// silu(gate) * up.  Without a gate, act >= 0 names an activation on the product (plain_act); -1: none.  32-bit
// accumulation in the order of k.
#define GG_BM 32
#define GG_BN 64
#define GG_BK 32
template <typename A, bool GATED>
__global__ void __launch_bounds__(256) moe_grouped_gemm_kernel(
        const A* __restrict__ a, int lda, const int* __restrict__ src, int src_div, const A* __restrict__ w,
        A* __restrict__ out, int ldo, const int* __restrict__ tiles, int N, int K, int act, float limit) {
    __shared__ float As[GG_BK][GG_BM + 1];
    __shared__ float Ws[GATED ? 2 : 1][GG_BK][GG_BN + 1];
    __shared__ int rowsrc[GG_BM];
    pdl_wait();
    pdl_trigger();
    const int* tl = tiles + 3 * (size_t)blockIdx.x;
    const int e = tl[0], first = tl[1], nrows = tl[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * GG_BN;
    const int tid = threadIdx.x;
    if (tid < GG_BM) rowsrc[tid] = tid < nrows ? (src ? src[first + tid] / src_div : first + tid) : -1;
    __syncthreads();
    const A* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    const int tr = tid / 16, tc = tid % 16;          // rows tr, tr + 16; columns tc + 16 j, j < 4
    float acc[2][4] = {}, acc2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int i = tid; i < GG_BM * GG_BK; i += 256) {
            const int r = i / GG_BK, k = i % GG_BK;
            const int row = rowsrc[r];
            As[k][r] = (row >= 0 && k0 + k < K) ? to_f32(a[(size_t)row * lda + k0 + k]) : 0.f;
        }
        for (int i = tid; i < GG_BN * GG_BK; i += 256) {
            const int n = i / GG_BK, k = i % GG_BK;
            const bool ok = n0 + n < N && k0 + k < K;
            Ws[0][k][n] = ok ? to_f32(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
            if (GATED) Ws[1][k][n] = ok ? to_f32(we[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < GG_BK; ++k) {
            const float a0 = As[k][tr], a1 = As[k][tr + 16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Ws[0][k][tc + 16 * j];
                acc[0][j] += a0 * b;
                acc[1][j] += a1 * b;
                if (GATED) {
                    const float b2 = Ws[1][k][tc + 16 * j];
                    acc2[0][j] += a0 * b2;
                    acc2[1][j] += a1 * b2;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = tr + 16 * i;
        if (r >= nrows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tc + 16 * j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = gated_act(v, acc2[i][j], act, limit);
            else if (act >= 0) v = plain_act(v, act);
            out[(size_t)(first + r) * ldo + n] = from_f32<A>(v);
        }
    }
}

extern "C" int rg_moe_grouped_gemm(const void* a, int lda, const int* src, int src_div, const void* w, void* out,
                                   int ldo, int dtype, const int* tiles, int max_tiles, int tile_rows, int N, int K,
                                   int gated, int act, float limit, void* stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (tile_rows != GG_BM || K < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_tiles, (N + GG_BN - 1) / GG_BN), block(256);
#define RG_GG(A, G) return rg_launch(moe_grouped_gemm_kernel<A, G>, grid, block, 0, s, 1, (const A*)a, lda, src, \
        src_div, (const A*)w, (A*)out, ldo, tiles, N, K, act, limit)
    if (dtype == RG_DTYPE_BF16 && gated) RG_GG(bf16, true);
    if (dtype == RG_DTYPE_BF16 && !gated) RG_GG(bf16, false);
    if (dtype == RG_DTYPE_F32 && gated) RG_GG(float, true);
    if (dtype == RG_DTYPE_F32 && !gated) RG_GG(float, false);
#undef RG_GG
    return RG_ERR_UNSUPPORTED;
}

// out[t] (32-bit) = sum_k weights[t, k] * (ids[t, k] < E ? y[pair_pos[t, k]] : x[t])  (+ shared[t]); weights null: all 1
template <typename A>
__global__ void moe_combine_kernel(const A* __restrict__ x, const A* __restrict__ y, const A* __restrict__ shared,
                                   const int* __restrict__ ids, const float* __restrict__ weights,
                                   const int* __restrict__ pair_pos, float* __restrict__ out, int W, int E, int top) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float csm[];                 // per choice: weight, row of y (-1: the token's own row)
    const int t = blockIdx.x;
    float* cw = csm;
    int* crow = reinterpret_cast<int*>(csm + top);
    for (int k = threadIdx.x; k < top; k += blockDim.x) {
        const size_t p = (size_t)t * top + k;
        cw[k] = weights ? weights[p] : 1.f;
        crow[k] = ids[p] < E ? pair_pos[p] : -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = 0.f;
        const float own = to_f32(x[(size_t)t * W + i]);
        for (int k = 0; k < top; ++k) {
            const int row = crow[k];
            v += cw[k] * (row >= 0 ? to_f32(y[(size_t)row * W + i]) : own);
        }
        if (shared) v += to_f32(shared[(size_t)t * W + i]);
        out[(size_t)t * W + i] = v;
    }
}

extern "C" int rg_moe_combine(const void* x, const void* y, const void* shared, int dtype, const int* ids,
                              const float* weights, const int* pair_pos, float* out, int T, int W, int E, int top,
                              void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = W >= 1024 ? 256 : 128;
    const size_t csmem = (size_t)top * 8;
    if (top < 1 || csmem > 48 * 1024) return RG_ERR_UNSUPPORTED;
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(moe_combine_kernel<bf16>, dim3(T), dim3(threads), csmem, s, 1, (const bf16*)x, (const bf16*)y,
                         (const bf16*)shared, ids, weights, pair_pos, out, W, E, top);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), csmem, s, 1, (const float*)x, (const float*)y,
                         (const float*)shared, ids, weights, pair_pos, out, W, E, top);
    return RG_ERR_UNSUPPORTED;
}

// out[pos] = a[src[pos] / src_div] for every place that has a pair (rows of K bfloat16 numbers, K % 8 == 0, copied
// 16 bytes at a time): the experts' input in expert order, for a product that reads its rows through TMA.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ a, int lda, const int* __restrict__ src, int src_div,
                                       bf16* __restrict__ out, int K) {
    pdl_wait();
    pdl_trigger();
    const int pos = blockIdx.x;
    const int pair = src[pos];
    if (pair < 0) return;
    const uint4* from = reinterpret_cast<const uint4*>(a + (size_t)(pair / src_div) * lda);
    uint4* to = reinterpret_cast<uint4*>(out + (size_t)pos * K);
    for (int i = threadIdx.x; i < (K >> 3); i += blockDim.x) to[i] = from[i];
}

// out[pos] = scale[src[pos]] * a[src[pos] / src_div]: the same rows, each times its pair's weight (32-bit product,
// one rounding), for experts whose weight multiplies their input.  Any K and either storage type.
template <typename A>
__global__ void moe_gather_scaled_rows_kernel(const A* __restrict__ a, int lda, const int* __restrict__ src, int src_div,
                                              const float* __restrict__ scale, A* __restrict__ out, int K) {
    pdl_wait();
    pdl_trigger();
    const int pos = blockIdx.x;
    const int pair = src[pos];
    if (pair < 0) return;
    const float f = scale[pair];
    const A* from = a + (size_t)(pair / src_div) * lda;
    A* to = out + (size_t)pos * K;
    for (int i = threadIdx.x; i < K; i += blockDim.x) to[i] = from_f32<A>(f * to_f32(from[i]));
}

// bfloat16 rows that start on 16-byte boundaries: eight numbers per thread and step.
__global__ void moe_gather_scaled_rows8_kernel(const bf16* __restrict__ a, int lda, const int* __restrict__ src,
                                               int src_div, const float* __restrict__ scale, bf16* __restrict__ out,
                                               int K) {
    pdl_wait();
    pdl_trigger();
    const int pos = blockIdx.x;
    const int pair = src[pos];
    if (pair < 0) return;
    const float f = scale[pair];
    const uint4* from = reinterpret_cast<const uint4*>(a + (size_t)(pair / src_div) * lda);
    uint4* to = reinterpret_cast<uint4*>(out + (size_t)pos * K);
    for (int i = threadIdx.x; i < (K >> 3); i += blockDim.x) {
        const uint4 v = from[i];
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __bfloat1622float2(v2[e]);
            o2[e] = __floats2bfloat162_rn(f * x.x, f * x.y);
        }
        to[i] = o;
    }
}

extern "C" int rg_moe_gather_scaled_rows(const void* a, int dtype, int lda, const int* src, int src_div,
                                         const float* scale, void* out, int P, int K, void* stream) {
    if (P <= 0) return 0;
    if (src_div < 1 || K < 1) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = K >= 2048 ? 256 : 128;
    if (dtype == RG_DTYPE_BF16 && (K & 7) == 0 && (lda & 7) == 0 && (((uintptr_t)a | (uintptr_t)out) & 15) == 0)
        return rg_launch(moe_gather_scaled_rows8_kernel, dim3(P), dim3(K >= 2048 ? 256 : (K >= 512 ? 64 : 32)), 0, s, 1,
                         (const bf16*)a, lda, src, src_div, scale, (bf16*)out, K);
    if (dtype == RG_DTYPE_BF16)
        return rg_launch(moe_gather_scaled_rows_kernel<bf16>, dim3(P), dim3(threads), 0, s, 1, (const bf16*)a, lda, src,
                         src_div, scale, (bf16*)out, K);
    if (dtype == RG_DTYPE_F32)
        return rg_launch(moe_gather_scaled_rows_kernel<float>, dim3(P), dim3(threads), 0, s, 1, (const float*)a, lda, src,
                         src_div, scale, (float*)out, K);
    return RG_ERR_UNSUPPORTED;
}

extern "C" int rg_moe_gather_rows(const void* a, int lda, const int* src, int src_div, void* out, int P, int K,
                                  void* stream) {
    if (P <= 0) return 0;
    if ((K & 7) || (lda & 7) || src_div < 1 || (((uintptr_t)a | (uintptr_t)out) & 15)) return RG_ERR_UNSUPPORTED;
    return rg_launch(moe_gather_rows_kernel, dim3(P), dim3(K >= 2048 ? 256 : 128), 0, (cudaStream_t)stream, 1,
                     (const bf16*)a, lda, src, src_div, (bf16*)out, K);
}

// ---------------------------------------------------------------------------------------------------
// The same product on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit accumulators): one block per
// (tile of BM places of one expert, 64 output columns), the expert's rows W[n0 .. n0 + 64) and the tile's
// gathered input rows streamed through a three-stage cp.async ring in steps of 64 along K.  With few places
// per expert (decode) the block is a weight-streaming product whose tile is mostly padding; with many
// (prompts) the products go to the tcgen05 kernel instead (gemm_tcgen05.cu, grouped).  GATED: gate and up rows side by side,
// silu(gate) * up in the epilogue, in 32-bit.  K and lda must be multiples of 8 (16-byte copies).
#include "mma.cuh"

#define GM_BN 64
#define GM_BK 64
#define GM_STAGES 3
#define GM_STRIDE (GM_BK + 8)

template <int BM, bool GATED>
__global__ void __launch_bounds__(BM == 128 ? 256 : 128) moe_grouped_gemm_mma_kernel(
        const bf16* __restrict__ a, int lda, const int* __restrict__ src, int src_div, const bf16* __restrict__ w,
        bf16* __restrict__ out, int ldo, const int* __restrict__ tiles, int N, int K, int act, float limit) {
    using namespace rgmma;
    constexpr int THREADS = BM == 128 ? 256 : 128;
    constexpr int WARPS_M = BM == 128 ? 4 : 2;                     // x 2 warps along the columns
    constexpr int WM = BM / WARPS_M;                               // rows per warp: 32 or 16
    constexpr int MI = WM / 16;
    constexpr int NB = GATED ? 2 : 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sA = reinterpret_cast<bf16*>(smem_raw);                  // [STAGES][BM][STRIDE]
    bf16* sB = sA + GM_STAGES * BM * GM_STRIDE;                    // [STAGES][NB][BN][STRIDE]
    __shared__ int rowsrc[BM];
    pdl_wait();
    pdl_trigger();
    const int* tl = tiles + 3 * (size_t)blockIdx.x;
    const int e = tl[0], first = tl[1], nrows = tl[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * GM_BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int r = tid; r < BM; r += THREADS) rowsrc[r] = r < nrows ? (src ? src[first + r] / src_div : first + r) : -1;
    __syncthreads();
    const bf16* we = w + (size_t)e * NB * N * K;
    const int ksteps = (K + GM_BK - 1) / GM_BK;

    auto load_stage = [&](int ks, int stage) {
        const int k0 = ks * GM_BK;
        bf16* dA = sA + stage * BM * GM_STRIDE;
        for (int i = tid; i < BM * (GM_BK / 8); i += THREADS) {
            const int r = i >> 3, c = (i & 7) * 8;
            const int row = rowsrc[r];
            const bool valid = row >= 0 && k0 + c < K;
            cp_async16(dA + r * GM_STRIDE + c, valid ? a + (size_t)row * lda + k0 + c : a, valid);
        }
        bf16* dB = sB + stage * NB * GM_BN * GM_STRIDE;
        for (int i = tid; i < NB * GM_BN * (GM_BK / 8); i += THREADS) {
            const int half = i / (GM_BN * 8), j = i - half * GM_BN * 8;
            const int n = j >> 3, c = (j & 7) * 8;
            const bool valid = n0 + n < N && k0 + c < K;
            cp_async16(dB + (half * GM_BN + n) * GM_STRIDE + c,
                       valid ? we + ((size_t)half * N + n0 + n) * K + k0 + c : we, valid);
        }
    };
#pragma unroll
    for (int s = 0; s < GM_STAGES - 1; ++s) {
        if (s < ksteps) load_stage(s, s);
        cp_async_commit();
    }
    const int wm = warp >> 1, wn = warp & 1;                       // warp tile: rows wm * WM, columns wn * 32
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
    float acc[NB][MI][4][4];
#pragma unroll
    for (int h = 0; h < NB; ++h)
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) { acc[h][mi][ni][0] = acc[h][mi][ni][1] = acc[h][mi][ni][2] = acc[h][mi][ni][3] = 0.f; }

    for (int ks = 0; ks < ksteps; ++ks) {
        cp_async_wait<GM_STAGES - 2>();
        __syncthreads();
        if (ks + GM_STAGES - 1 < ksteps) load_stage(ks + GM_STAGES - 1, (ks + GM_STAGES - 1) % GM_STAGES);
        cp_async_commit();
        const bf16* cA = sA + (ks % GM_STAGES) * BM * GM_STRIDE;
        const bf16* cB = sB + (ks % GM_STAGES) * NB * GM_BN * GM_STRIDE;
#pragma unroll
        for (int kk = 0; kk < GM_BK / 16; ++kk) {
            uint32_t af[MI][4];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
                ldmatrix_x4(af[mi], cA + (wm * WM + mi * 16 + a_row) * GM_STRIDE + kk * 16 + a_col);
#pragma unroll
            for (int h = 0; h < NB; ++h) {
#pragma unroll
                for (int n2 = 0; n2 < 2; ++n2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, cB + (h * GM_BN + wn * 32 + n2 * 16 + b_row) * GM_STRIDE + kk * 16 + b_col);
#pragma unroll
                    for (int mi = 0; mi < MI; ++mi) {
                        mma_bf16(acc[h][mi][2 * n2], af[mi], b[0], b[1]);
                        mma_bf16(acc[h][mi][2 * n2 + 1], af[mi], b[2], b[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * WM + mi * 16 + g + half * 8;
            if (r >= nrows) continue;
            bf16* orow = out + (size_t)(first + r) * ldo;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int n = n0 + wn * 32 + ni * 8 + tq * 2 + c;
                    if (n >= N) continue;
                    float v = acc[0][mi][ni][half * 2 + c];
                    if (GATED) v = gated_act(v, acc[NB - 1][mi][ni][half * 2 + c], act, limit);
                    else if (act >= 0) v = plain_act(v, act);
                    orow[n] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}

template <typename KF> static int gm_allow_smem(KF kernel, size_t bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// tile_rows: 32, the tile size `moe_align` was given.
extern "C" int rg_moe_grouped_gemm_mma(const void* a, int lda, const int* src, int src_div, const void* w, void* out,
                                       int ldo, const int* tiles, int max_tiles, int tile_rows, int N, int K,
                                       int gated, int act, float limit, void* stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (tile_rows != 32 || K < 8 || (K & 7) || (lda & 7) || src_div < 1) return RG_ERR_UNSUPPORTED;
    if (((uintptr_t)a | (uintptr_t)w) & 15) return RG_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(max_tiles, (N + GM_BN - 1) / GM_BN);
    int e;
#define RG_GM(BM, G) { const size_t smem = (size_t)GM_STAGES * (BM + (G ? 2 : 1) * GM_BN) * GM_STRIDE * 2; \
        e = gm_allow_smem(moe_grouped_gemm_mma_kernel<BM, G>, smem); if (e) return e; \
        return rg_launch(moe_grouped_gemm_mma_kernel<BM, G>, grid, dim3(BM == 128 ? 256 : 128), smem, s, 1, \
                         (const bf16*)a, lda, src, src_div, (const bf16*)w, (bf16*)out, ldo, tiles, N, K, act, limit); }
    if (gated) RG_GM(32, true)
    RG_GM(32, false)
#undef RG_GM
}
