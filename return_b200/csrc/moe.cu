// Mixture of experts: the router's choice, the experts' products for (token, chosen expert) pairs, the gated unit
// with a capped gate, and the weighted sum.
//
// A step's tokens each choose `top` of E experts.  Pair i = t * top + k is token t's k-th choice (in the order of
// falling score); expert_of[i] names its expert, weight[i] its share.  Everything is worked out on the device from
// the router's logits, with grids that depend on the number of tokens only, so a step can be captured in a graph.
#include "common.cuh"

// ---------------------------------------------------------------- the router's choice
// One warp a token.  s = softmax(z + bias) over all experts (float32; the bias per expert may be absent).  With groups > 1 the experts form `groups` equal
// runs of neighbours, a group's score is its largest s, and only experts of the `keep` best groups can be chosen.
// The `top` largest s among those are chosen (the lower index on a tie); weight = s / (sum of the chosen s + tiny),
// which with tiny = 0 is the softmax over the chosen logits alone.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, int* __restrict__ expert_of,
                 float* __restrict__ weight, int T, int E, int top, int groups, int keep, float tiny, int score_fn,
                 int group_top, float out_scale) {
    extern __shared__ float route_smem[];                 // per warp: E scores, then `groups` group scores
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s = route_smem + (size_t)warp * (E + groups);
    float* gs = s + E;
    const float* zr = z + (size_t)t * ldz;
    if (score_fn == 1) {                                  // every expert scored by itself: the logistic of its logit
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-(zr[e] + (bias ? bias[e] : 0.f))));
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) {
            const float v = zr[e] + (bias ? bias[e] : 0.f);    // the logit with its bias waits in s[e] for the second pass
            s[e] = v;
            m = fmaxf(m, v);
        }
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(s[e] - m);
            s[e] = v;
            sum += v;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) s[e] *= inv;
    }
    __syncwarp();
    const int gsize = E / groups;
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            float b = -1.f, b2 = -1.f;                        // the group's two best scores
            for (int e = g * gsize; e < (g + 1) * gsize; ++e) {
                const float v = s[e];
                if (v > b) { b2 = b; b = v; } else if (v > b2) { b2 = v; }
            }
            gs[g] = (group_top >= 2 && b2 >= 0.f) ? b + b2 : b;
        }
        __syncwarp();
        for (int r = 0; r < keep; ++r) {                  // the best group not yet kept becomes -2: kept
            float bv = -1.f;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] > bv) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            __syncwarp();
            if (lane == 0 && bi < groups) gs[bi] = -2.f;
            __syncwarp();
        }
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const bool open = groups <= 1 || gs[e / gsize] == -2.f;
            if (open && s[e] > bv) { bv = s[e]; bi = e; }
        }
        warp_argmax(bv, bi);
        __syncwarp();
        if (lane == 0) {
            expert_of[(size_t)t * top + k] = bi < E ? bi : 0;
            weight[(size_t)t * top + k] = bv;             // the score for now; divided below
            if (bi < E) s[bi] = -1.f;
        }
        total += bv;
        __syncwarp();
    }
    const float scale = out_scale / (total + tiny);
    __syncwarp();
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= scale;
}

RB_EXPORT int rb_moe_route(const float* z, int ldz, const float* bias, int* expert_of, float* weight, int T, int E, int top,
                           int groups, int keep, float tiny, int score_fn, int group_top, float out_scale, cudaStream_t st) {
    if (T <= 0) return 0;
    if (score_fn < 0 || score_fn > 1 || group_top < 1 || group_top > 2) return (int)cudaErrorInvalidValue;
    if (groups < 1 || E % groups || top < 1 || top > E || keep < 1 || keep > groups || (long long)keep * (E / groups) < top)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)4 * (E + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(moe_route_kernel, dim3((T + 3) / 4), dim3(128), smem, st, z, ldz, bias, expert_of, weight, T, E, top,
                         groups, keep, tiny, score_fn, group_top, out_scale);
}

// ---------------------------------------------------------------- a pair's product, weights streamed
// out[i, n] = sum_k x[i / in_div, k] * W[expert_of[i]][n, k] for every pair i: the form for few pairs (decoded tokens)
// and the float32 path.  One CTA takes one pair and a run of output rows; a warp an output row at a time, the lanes
// striding k, so every sum has one order whatever else the step holds.  W: [E, N, K] contiguous.
template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
moe_pair_linear_kernel(const TA* __restrict__ x, int ldx, int in_div, const TA* __restrict__ W, const int* __restrict__ expert_of,
                       TO* __restrict__ out, int ldo, int N, int K, int rows_per_cta) {
    extern __shared__ float xs[];                         // K floats
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const TA* xr = x + (size_t)(i / in_div) * ldx;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32(xr[k]);
    __syncthreads();
    const TA* We = W + (size_t)expert_of[i] * N * K;
    const int n0 = blockIdx.y * rows_per_cta;
    const int n1 = min(N, n0 + rows_per_cta);
    for (int n = n0 + warp; n < n1; n += nwarps) {
        const TA* wr = We + (size_t)n * K;
        float acc = 0.f;
        for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], to_f32(wr[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) out[(size_t)i * ldo + n] = from_f32<TO>(acc);
    }
}

// The bfloat16 form for rows of whole 16-byte pieces: a lane reads eight weights at a time from each of four output
// rows (four loads in flight, 512 bytes a row and step over the warp), the token's row waits in shared memory as
// float32.  Eight warps share 64 output rows; the sums keep one order (a lane's pieces in turn, then the butterfly).
__global__ void __launch_bounds__(256)
moe_pair_linear_vec_kernel(const bf16* __restrict__ x, int ldx, int in_div, const bf16* __restrict__ W,
                           const int* __restrict__ expert_of, bf16* __restrict__ out, int ldo, int N, int K) {
    extern __shared__ __align__(16) float xs[];           // K floats
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bf16* xr = x + (size_t)(i / in_div) * ldx;
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + k);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            xs[k + 2 * j] = f.x;
            xs[k + 2 * j + 1] = f.y;
        }
    }
    __syncthreads();
    const bf16* We = W + (size_t)expert_of[i] * N * K;
    const int n_base = blockIdx.y * 64 + warp * 8;
#pragma unroll 1
    for (int r0 = 0; r0 < 8; r0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* wr[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wr[j] = We + (size_t)min(n_base + r0 + j, N - 1) * K;      // a row past the end reads the last one
        for (int k = lane * 8; k < K; k += 256) {
            uint4 wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const uint4*>(wr[j] + k);
            const float4 xa = *reinterpret_cast<const float4*>(xs + k), xb = *reinterpret_cast<const float4*>(xs + k + 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&wv[j]);
                const float2 w0 = __bfloat1622float2(p[0]), w1 = __bfloat1622float2(p[1]);
                const float2 w2 = __bfloat1622float2(p[2]), w3 = __bfloat1622float2(p[3]);
                acc[j] = fmaf(xa.x, w0.x, acc[j]); acc[j] = fmaf(xa.y, w0.y, acc[j]);
                acc[j] = fmaf(xa.z, w1.x, acc[j]); acc[j] = fmaf(xa.w, w1.y, acc[j]);
                acc[j] = fmaf(xb.x, w2.x, acc[j]); acc[j] = fmaf(xb.y, w2.y, acc[j]);
                acc[j] = fmaf(xb.z, w3.x, acc[j]); acc[j] = fmaf(xb.w, w3.y, acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float v = warp_sum(acc[j]);
            const int n = n_base + r0 + j;
            if (lane == 0 && n < N) out[(size_t)i * ldo + n] = __float2bfloat16_rn(v);
        }
    }
    pdl_trigger_late();
}

RB_EXPORT int rb_moe_pair_linear(const void* x, int ldx, int in_div, const void* W, const int* expert_of, void* out, int ldo,
                                 int act_dtype, int pairs, int N, int K, cudaStream_t st) {
    if (pairs <= 0 || N <= 0) return 0;
    const int rows_per_cta = 64;
    dim3 grid(pairs, (N + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (act_dtype == RB_BF16 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0)
        return rb_launch_pdl(moe_pair_linear_vec_kernel, grid, dim3(256), smem, st, (const bf16*)x, ldx, in_div, (const bf16*)W,
                             expert_of, (bf16*)out, ldo, N, K);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(moe_pair_linear_kernel<float, float>, grid, dim3(256), smem, st, (const float*)x, ldx, in_div,
                             (const float*)W, expert_of, (float*)out, ldo, N, K, rows_per_cta);
    return rb_launch_pdl(moe_pair_linear_kernel<bf16, bf16>, grid, dim3(256), smem, st, (const bf16*)x, ldx, in_div,
                         (const bf16*)W, expert_of, (bf16*)out, ldo, N, K, rows_per_cta);
}

// ---------------------------------------------------------------- the gated unit with a capped gate
// in[r] = [gate (F numbers) | up (F numbers)];  g = min(gate, limit), u = clamp(up, -limit, limit);
// out[r, f] = g * sigmoid(alpha * g) * (u + shift).  float32 arithmetic, one rounding at the store.  An infinite limit,
// alpha = 1 and shift = 0 make it silu(gate) * up.
template <typename TA>
__global__ void clamped_glu_kernel(const TA* __restrict__ in, int ldi, TA* __restrict__ out, int ldo, int F, float limit,
                                   float alpha, float shift, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / F;
        const int f = (int)(e % F);
        const float g = fminf(to_f32(in[r * ldi + f]), limit);
        const float u = fminf(fmaxf(to_f32(in[r * ldi + F + f]), -limit), limit);
        out[r * ldo + f] = from_f32<TA>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

// bfloat16 with F a multiple of 8: eight outputs (two 16-byte loads, one store) a thread and step.
__global__ void clamped_glu_bf16x8_kernel(const bf16* __restrict__ in, int ldi, bf16* __restrict__ out, int ldo, int F8,
                                          float limit, float alpha, float shift, unsigned total) {
    pdl_launch_dependents();
    pdl_wait();
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const unsigned r = e / F8, f = (e - r * F8) * 8;
        const uint4 gv = *reinterpret_cast<const uint4*>(in + (size_t)r * ldi + f);
        const uint4 uv = *reinterpret_cast<const uint4*>(in + (size_t)r * ldi + F8 * 8 + f);
        const bf16* g8 = reinterpret_cast<const bf16*>(&gv);
        const bf16* u8 = reinterpret_cast<const bf16*>(&uv);
        uint4 ov;
        bf16* o8 = reinterpret_cast<bf16*>(&ov);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float g = fminf(__bfloat162float(g8[k]), limit);
            const float u = fminf(fmaxf(__bfloat162float(u8[k]), -limit), limit);
            o8[k] = __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + shift));
        }
        *reinterpret_cast<uint4*>(out + (size_t)r * ldo + f) = ov;
    }
}

RB_EXPORT int rb_clamped_glu(const void* in, int ldi, void* out, int ldo, int act_dtype, int rows, int F, float limit,
                             float alpha, float shift, cudaStream_t st) {
    const long long total = (long long)rows * F;
    if (total <= 0) return 0;
    if (act_dtype == RB_BF16 && F % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)in % 16) == 0 &&
        ((uintptr_t)out % 16) == 0 && total / 8 < 0x7fffffffLL) {
        const unsigned items = (unsigned)(total / 8);
        const int nblocks = (int)min((unsigned)(148 * 16), (items + 255) / 256);
        return rb_launch_pdl(clamped_glu_bf16x8_kernel, dim3(nblocks), dim3(256), 0, st, (const bf16*)in, ldi, (bf16*)out, ldo,
                             F / 8, limit, alpha, shift, items);
    }
    const int blocks = (int)min((long long)4096, (total + 255) / 256);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(clamped_glu_kernel<float>, dim3(blocks), dim3(256), 0, st, (const float*)in, ldi, (float*)out, ldo, F,
                             limit, alpha, shift, total);
    return rb_launch_pdl(clamped_glu_kernel<bf16>, dim3(blocks), dim3(256), 0, st, (const bf16*)in, ldi, (bf16*)out, ldo, F, limit,
                         alpha, shift, total);
}

// ---------------------------------------------------------------- the weighted sum of a token's experts
// out[t, :] = sum_k weight[t, k] * y[row_of ? row_of[t * top + k] : t * top + k, :]  (+ shared[t, :]), k ascending, float32
// sums.  row_of: where a pair's row lies when the pairs were put in the order of their experts.
template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ weight,
                                   const TA* __restrict__ shared, TA* __restrict__ out, int H, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int pair = t * top + k;
            const size_t row = row_of ? (size_t)row_of[pair] : (size_t)pair;
            acc = fmaf(weight[pair], to_f32(y[row * H + i]), acc);
        }
        if (shared != nullptr) acc += to_f32(shared[(size_t)t * H + i]);
        out[(size_t)t * H + i] = from_f32<TA>(acc);
    }
}

RB_EXPORT int rb_moe_combine(const void* y, const int* row_of, const float* weight, const void* shared, void* out,
                             int act_dtype, int T, int H, int top, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)y, row_of, weight,
                             (const float*)shared, (float*)out, H, top);
    return rb_launch_pdl(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, st, (const bf16*)y, row_of, weight,
                         (const bf16*)shared, (bf16*)out, H, top);
}

// ---------------------------------------------------------------- the pairs in the order of their experts
// A counting sort by one CTA: offsets[e] .. offsets[e + 1] is expert e's run of places, pair_at[place] the pair that
// stands there, place_of[pair] its inverse.  Which of an expert's pairs gets which place is left to the atomics: every
// row of the products below is worked out by itself, so the places change no result.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ expert_of, int pairs, int E, int* __restrict__ offsets, int* __restrict__ pair_at,
                int* __restrict__ place_of) {
    extern __shared__ int sort_smem[];                    // E counts, then E cursors
    int* counts = sort_smem;
    int* cursor = sort_smem + E;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&counts[expert_of[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[E] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int place = atomicAdd(&cursor[expert_of[i]], 1);
        pair_at[place] = i;
        place_of[i] = place;
    }
}

RB_EXPORT int rb_moe_sort(const int* expert_of, int pairs, int E, int* offsets, int* pair_at, int* place_of, cudaStream_t st) {
    if (pairs <= 0) return 0;
    const size_t smem = (size_t)2 * E * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), smem, st, expert_of, pairs, E, offsets, pair_at, place_of);
}

// ---------------------------------------------------------------- the experts' products on the tensor cores
// C[place, n] = sum_k A[row(place), k] * W[e][n, k] for every place of expert e's run, bfloat16 in, float32
// accumulation (mma.sync m16n8k16), bfloat16 out.  row(place) = pair_at[place] / in_div when pair_at is given (the
// first product reads the tokens' rows where they lie), else the place itself (the second reads what the first left).
// A CTA owns a tile of 64 places of one expert x 128 output columns; it finds its expert by walking the offsets,
// and leaves at once if the step has fewer tiles than the grid (which is sized for the worst case, so that nothing
// about a launch depends on the router's choice).  Operands come in through a three-stage cp.async pipeline; rows
// behind an expert's run and columns behind K are filled with zeros.  K % 8 == 0; rows 16-byte aligned.
#define GG_BM 64
#define GG_BN 128
#define GG_BK 32
#define GG_LD 40                                           // padded row of a tile in shared memory (elements)
#define GG_STAGES 3

__device__ __forceinline__ void gg_cp16(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void gg_ldsm4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void gg_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256)
moe_grouped_gemm_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ pair_at, int in_div,
                        const bf16* __restrict__ W, const int* __restrict__ offsets, int E, bf16* __restrict__ C, int ldc,
                        int N, int K) {
    __shared__ __align__(16) bf16 sA[GG_STAGES][GG_BM * GG_LD];
    __shared__ __align__(16) bf16 sB[GG_STAGES][GG_BN * GG_LD];
    __shared__ int s_tile[3];                             // expert, first place of the tile, places in it
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int left = blockIdx.x, e = 0, found = -1, first = 0, count = 0;
        for (; e < E; ++e) {
            const int lo = offsets[e], n = offsets[e + 1] - lo;
            const int tiles = (n + GG_BM - 1) / GG_BM;
            if (left < tiles) { found = e; first = lo + left * GG_BM; count = min(GG_BM, n - left * GG_BM); break; }
            left -= tiles;
        }
        s_tile[0] = found; s_tile[1] = first; s_tile[2] = count;
    }
    __syncthreads();
    const int e = s_tile[0];
    if (e < 0) return;
    const int first = s_tile[1], rows = s_tile[2];
    const int n0 = blockIdx.y * GG_BN;
    const bf16* We = W + (size_t)e * N * K;

    // what this thread copies every stage: one 16-byte piece of A, two of B
    const int a_row = tid >> 2, a_ch = tid & 3;
    const bool a_ok = a_row < rows;
    const int a_place = first + a_row;
    const size_t a_src = a_ok ? (size_t)(pair_at ? pair_at[a_place] / in_div : a_place) * lda : 0;
    const int b_row0 = tid >> 2, b_row1 = b_row0 + 64, b_ch = tid & 3;
    const bool b_ok0 = n0 + b_row0 < N, b_ok1 = n0 + b_row1 < N;
    const int kt_count = (K + GG_BK - 1) / GG_BK;
    auto load_stage = [&](int stage, int kt) {
        const int k = kt * GG_BK + a_ch * 8;
        const bool kin = k < K;
        gg_cp16(&sA[stage][a_row * GG_LD + a_ch * 8], A + a_src + (kin ? k : 0), a_ok && kin);
        gg_cp16(&sB[stage][b_row0 * GG_LD + b_ch * 8], We + (size_t)(b_ok0 ? n0 + b_row0 : 0) * K + (kin ? k : 0), b_ok0 && kin);
        gg_cp16(&sB[stage][b_row1 * GG_LD + b_ch * 8], We + (size_t)(b_ok1 ? n0 + b_row1 : 0) * K + (kin ? k : 0), b_ok1 && kin);
    };
    for (int s = 0; s < GG_STAGES - 1; ++s) {
        if (s < kt_count) load_stage(s, s);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;   // the warp's 32 x 32 part of the tile
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    for (int kt = 0; kt < kt_count; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(GG_STAGES - 2));
        __syncthreads();                                  // stage kt has landed; everyone is done with stage kt - 1
        if (kt + GG_STAGES - 1 < kt_count) load_stage((kt + GG_STAGES - 1) % GG_STAGES, kt + GG_STAGES - 1);
        asm volatile("cp.async.commit_group;\n" ::);
        const bf16* tA = sA[kt % GG_STAGES];
        const bf16* tB = sB[kt % GG_STAGES];
#pragma unroll
        for (int ks = 0; ks < GG_BK / 16; ++ks) {
            unsigned af[2][4], bfr[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                gg_ldsm4(af[i], tA + (wm + i * 16 + (lane & 15)) * GG_LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < 2; ++j)
                gg_ldsm4(bfr[j], tB + (wn + j * 16 + (lane & 7) + ((lane >> 4) << 3)) * GG_LD + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    gg_mma(acc[i][2 * j], af[i], bfr[j][0], bfr[j][1]);
                    gg_mma(acc[i][2 * j + 1], af[i], bfr[j][2], bfr[j][3]);
                }
        }
    }
    pdl_trigger_late();
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm + i * 16 + g + half * 8;
            if (r >= rows) continue;
            bf16* crow = C + (size_t)(first + r) * ldc;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + 2 * t4;
                if (n < N) crow[n] = __float2bfloat16_rn(acc[i][j][half * 2]);
                if (n + 1 < N) crow[n + 1] = __float2bfloat16_rn(acc[i][j][half * 2 + 1]);
            }
        }
}

RB_EXPORT int rb_moe_grouped_gemm(const void* A, int lda, const int* pair_at, int in_div, const void* W, const int* offsets,
                                  int E, void* C, int ldc, int places, int N, int K, cudaStream_t st) {
    if (places <= 0 || N <= 0) return 0;
    if (K % 8 || lda % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return (int)cudaErrorInvalidValue;
    dim3 grid((places + GG_BM - 1) / GG_BM + E, (N + GG_BN - 1) / GG_BN);
    return rb_launch_pdl(moe_grouped_gemm_kernel, grid, dim3(256), 0, st, (const bf16*)A, lda, pair_at, in_div, (const bf16*)W,
                         offsets, E, (bf16*)C, ldc, N, K);
}

// ---------------------------------------------------------------- the tokens' rows in the order of the places
// out[place, :] = x[pair_at[place] / in_div, :], 16 bytes a thread and step: what a product that wants its rows
// contiguous (operands by TMA) reads.  Rows of `bytes` bytes, a multiple of 16.
__global__ void moe_gather_rows_kernel(const unsigned char* __restrict__ x, long long ldx_bytes, const int* __restrict__ pair_at,
                                       int in_div, unsigned char* __restrict__ out, int bytes) {
    pdl_launch_dependents();
    pdl_wait();
    const int place = blockIdx.x;
    const unsigned char* src = x + (size_t)(pair_at[place] / in_div) * ldx_bytes;
    unsigned char* dst = out + (size_t)place * bytes;
    for (int b = threadIdx.x * 16; b < bytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(src + b);
}

RB_EXPORT int rb_moe_gather_rows(const void* x, long long ldx_bytes, const int* pair_at, int in_div, void* out, int bytes,
                                 int places, cudaStream_t st) {
    if (places <= 0) return 0;
    if (bytes % 16 || ldx_bytes % 16 || ((uintptr_t)x % 16) || ((uintptr_t)out % 16)) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(moe_gather_rows_kernel, dim3(places), dim3(128), 0, st, (const unsigned char*)x, ldx_bytes, pair_at,
                         in_div, (unsigned char*)out, bytes);
}
