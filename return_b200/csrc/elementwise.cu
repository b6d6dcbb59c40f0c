// Embedding gather, fused residual-add + RMSNorm, SwiGLU, row gather.
//
// The residual stream is float32 in both precisions; the "delta" a block adds to it and the
// normalised activations are in the activation dtype (float32 or bfloat16).  All arithmetic
// is float32 with one rounding at the store, as in the reference's Triton kernels
// (rollout/fused.py:6-17 for the norm, rollout/fused.py:103-127 for SwiGLU).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// stream[t, c, :] = scale * float(table[tokens[t], :]) for each of `copies` copies c (a model that keeps several
// residual streams starts them all from the embedded token).  A token id outside [0, V) writes NaN so that the
// fault shows in the logits instead of reading foreign memory.
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                 float* __restrict__ stream, int H, int V, float scale, int copies) {
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* dst = stream + (size_t)t * copies * H;
    const bool bad = id < 0 || id >= V;
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = bad ? __int_as_float(0x7fc00000) : to_f32(src[i]) * scale;
        for (int c = 0; c < copies; ++c) dst[(size_t)c * H + i] = v;
    }
}

// Sixteen bytes of the table per thread and iteration, for rows whose length allows it.
template <typename TW>
__global__ void embedding_vec_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                     float* __restrict__ stream, int H, int V, float scale, int copies) {
    constexpr int E = 16 / sizeof(TW);
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* dst = stream + (size_t)t * copies * H;
    const bool bad = id < 0 || id >= V;
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    for (int i = threadIdx.x * E; i < H; i += blockDim.x * E) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
        const TW* e = reinterpret_cast<const TW*>(&raw);
        float out[E];
#pragma unroll
        for (int k = 0; k < E; ++k) out[k] = bad ? __int_as_float(0x7fc00000) : to_f32(e[k]) * scale;
        for (int c = 0; c < copies; ++c) {
#pragma unroll
            for (int k = 0; k < E; k += 4)
                *reinterpret_cast<float4*>(dst + (size_t)c * H + i + k) = make_float4(out[k], out[k + 1], out[k + 2], out[k + 3]);
        }
    }
}

RB_EXPORT int rb_embedding(const void* table, int table_dtype, const int* tokens, float* stream,
                           int T, int H, int V, float scale, int copies, cudaStream_t st) {
    if (T <= 0) return 0;
    if (copies < 1) return (int)cudaErrorInvalidValue;
    const int threads = H >= 1024 ? 256 : 128;
    const bool aligned = ((uintptr_t)table % 16) == 0 && ((uintptr_t)stream % 16) == 0;
    if (table_dtype == RB_F32) {
        if (aligned && H % 4 == 0)
            return rb_launch_pdl(embedding_vec_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)table, tokens, stream, H, V, scale, copies);
        else
            embedding_kernel<float><<<T, threads, 0, st>>>((const float*)table, tokens, stream, H, V, scale, copies);
    } else {
        if (aligned && H % 8 == 0)
            return rb_launch_pdl(embedding_vec_kernel<bf16>, dim3(T), dim3(threads), 0, st, (const bf16*)table, tokens, stream, H, V, scale, copies);
        else
            embedding_kernel<bf16><<<T, threads, 0, st>>>((const bf16*)table, tokens, stream, H, V, scale, copies);
    }
    return rb_launch_status();
}

// ---------------------------------------------------------------- residual add + RMSNorm
// x = stream[row] (+ delta[row]);  if rows == nullptr the sum is written back to the stream;
// out[blockIdx.x] = x * rsqrt(mean(x^2) + eps) * (offset + w).
// With `rows` the kernel normalises only the listed rows (the rows whose logits are wanted)
// and leaves the stream untouched, so a row may be listed twice.
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ stream, const TA* __restrict__ delta,
                                   const int* __restrict__ rows, const void* __restrict__ w,
                                   int w_dtype, float eps, float offset, TA* __restrict__ out, int H) {
    extern __shared__ float smem[];
    float* xrow = smem;          // H floats
    float* scratch = smem + H;   // 33 floats
    const int orow = blockIdx.x;
    const int irow = rows ? rows[orow] : orow;
    float* s = stream + (size_t)irow * H;
    const TA* d = delta ? delta + (size_t)irow * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = s[i];
        if (d) x += to_f32(d[i]);
        xrow[i] = x;
        if (d && !rows) s[i] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)orow * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f32<TA>(xrow[i] * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

// The same, four elements per vector and up to VPT vectors per thread held in registers: every
// load of a row is in flight at once, which is what a step of a few rows needs (it is bound by
// the latency of one trip to memory, not by bandwidth).  Needs H % 4 == 0 and H <= 4 * VPT * threads.
template <typename TA> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&a);
        raw.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TA, typename TW, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ stream, const TA* __restrict__ delta,
                                       const int* __restrict__ rows, const TW* __restrict__ w,
                                       float eps, float offset, TA* __restrict__ out, int H) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int orow = blockIdx.x;
    const int nvec = H >> 2;
    float4 x[VPT], wv[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {                      // the norm weight is nobody's output: read it early
        const int i = threadIdx.x + v * blockDim.x;
        wv[v] = i < nvec ? Vec4<TW>::load(w + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const int irow = rows ? rows[orow] : orow;
    float* s = stream + (size_t)irow * H;
    const TA* d = delta ? delta + (size_t)irow * H : nullptr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        x[v] = i < nvec ? Vec4<float>::load(s + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (d) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * blockDim.x;
            if (i < nvec) {
                const float4 dv = Vec4<TA>::load(d + 4 * i);
                x[v].x += dv.x; x[v].y += dv.y; x[v].z += dv.z; x[v].w += dv.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
    if (d && !rows) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * blockDim.x;
            if (i < nvec) Vec4<float>::store(s + 4 * i, x[v]);
        }
    }
    pdl_trigger_late();
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)orow * H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (i < nvec)
            Vec4<TA>::store(o + 4 * i, make_float4(x[v].x * rstd * (offset + wv[v].x), x[v].y * rstd * (offset + wv[v].y),
                                                   x[v].z * rstd * (offset + wv[v].z), x[v].w * rstd * (offset + wv[v].w)));
    }
}

template <typename TA, typename TW>
static int launch_add_rmsnorm_vec(float* stream, const void* delta, const int* rows, const void* w, float eps,
                                  float offset, void* out, int n_rows, int H, cudaStream_t st) {
    const int nvec = H >> 2;
    int threads = 128;
    while (threads < 1024 && threads * 4 < nvec) threads <<= 1;
    if (threads >= nvec)
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 1>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    else if (threads * 2 >= nvec)
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 2>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    else
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 4>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    return rb_launch_status();
}

RB_EXPORT int rb_add_rmsnorm(float* stream, const void* delta, const int* rows, const void* w,
                             int w_dtype, float eps, float offset, void* out, int act_dtype,
                             int n_rows, int H, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const bool aligned = ((uintptr_t)stream % 16) == 0 && ((uintptr_t)delta % 16) == 0 &&
                         ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0;
    if (aligned && H % 4 == 0 && H <= 4 * 4 * 1024) {
        if (act_dtype == RB_F32 && w_dtype == RB_F32) return launch_add_rmsnorm_vec<float, float>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        if (act_dtype == RB_F32) return launch_add_rmsnorm_vec<float, bf16>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        if (w_dtype == RB_F32) return launch_add_rmsnorm_vec<bf16, float>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        return launch_add_rmsnorm_vec<bf16, bf16>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
    }
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    int threads = 128;
    while (threads < 1024 && threads * 8 < H) threads <<= 1;
    if (act_dtype == RB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<float><<<n_rows, threads, smem, st>>>(stream, (const float*)delta, rows, w, w_dtype,
                                                                eps, offset, (float*)out, H);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<bf16><<<n_rows, threads, smem, st>>>(stream, (const bf16*)delta, rows, w, w_dtype,
                                                               eps, offset, (bf16*)out, H);
    }
    return rb_launch_status();
}

// ---------------------------------------------------------------- plain RMSNorm over the last dim
// y[r, :] = x[r, :] * rsqrt(mean(x^2) + eps) * (offset + w), rows of length N (any N), one warp a row.
// The stand-alone form of the norm, used for kernel tests and by parts that need no residual.
template <typename TA>
__global__ void rmsnorm_rows_kernel(const TA* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                    float eps, float offset, TA* __restrict__ y, int rows, int N, int ldx, int ldy) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const TA* xr = x + (size_t)warp * ldx;
    float ss = 0.f;
    for (int i = lane; i < N; i += 32) { float v = to_f32(xr[i]); ss += v * v; }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)N + eps);
    TA* yr = y + (size_t)warp * ldy;
    for (int i = lane; i < N; i += 32)
        yr[i] = from_f32<TA>(to_f32(xr[i]) * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

// rows of length N that lie ldx (ldy) elements apart: a run of columns of a wider buffer
RB_EXPORT int rb_rmsnorm_rows_ld(const void* x, int ldx, const void* w, int w_dtype, float eps, float offset, void* y, int ldy,
                                 int act_dtype, int rows, int N, cudaStream_t st) {
    if (rows <= 0) return 0;
    const int threads = 128, per_block = threads / 32;
    const int blocks = (rows + per_block - 1) / per_block;
    if (act_dtype == RB_F32)
        rmsnorm_rows_kernel<float><<<blocks, threads, 0, st>>>((const float*)x, w, w_dtype, eps, offset, (float*)y, rows, N, ldx, ldy);
    else
        rmsnorm_rows_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)x, w, w_dtype, eps, offset, (bf16*)y, rows, N, ldx, ldy);
    return rb_launch_status();
}

RB_EXPORT int rb_rmsnorm_rows(const void* x, const void* w, int w_dtype, float eps, float offset, void* y,
                              int act_dtype, int rows, int N, cudaStream_t st) {
    return rb_rmsnorm_rows_ld(x, N, w, w_dtype, eps, offset, y, N, act_dtype, rows, N, st);
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gate) * up.  gu is [T, 2I].  block == 0: gate columns [0, I), up columns [I, 2I)
// (the reference's concatenation, rollout/monkey_patch/qwen3.py:99-105).  block == 8: columns come in
// blocks of 8 gate then 8 up (the layout that lets a matrix product's epilogue do this step).
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int T, int I, int block) {
    const size_t total = (size_t)T * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx - t * I;
        const size_t gi = block ? (i / block) * 2 * block + i % block : i;
        const size_t ui = block ? gi + block : I + i;
        const float g = to_f32(gu[t * 2 * I + gi]);
        const float u = to_f32(gu[t * 2 * I + ui]);
        out[idx] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 with I a multiple of 8: eight elements (16 bytes) per thread, two such pieces in flight.
// The exponential and the division are the fast float32 forms (a few units in the last place, far
// below the rounding to bfloat16 that follows): with the accurate ones the kernel is bound by
// instruction issue, not by memory.
__device__ __forceinline__ uint4 swiglu8(const uint4 gv, const uint4 uv) {
    const bf16* g = (const bf16*)&gv;
    const bf16* u = (const bf16*)&uv;
    uint4 ov;
    bf16* o = (bf16*)&ov;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float gf = __bfloat162float(g[k]);
        o[k] = __float2bfloat16_rn(__fdividef(gf, 1.0f + __expf(-gf)) * __bfloat162float(u[k]));
    }
    return ov;
}

__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int T, int I, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int I8 = I >> 3;
    const size_t total = (size_t)T * I8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += 2 * stride) {
        const size_t idx2 = idx + stride;
        const bool two = idx2 < total;
        const size_t t = idx / I8, i = (idx - t * I8) << 3;
        const size_t t2 = two ? idx2 / I8 : t, i2 = two ? (idx2 - t2 * I8) << 3 : i;
        const uint4 gv = *(const uint4*)(gu + t * 2 * I + (block ? 2 * i : i));
        const uint4 uv = *(const uint4*)(gu + t * 2 * I + (block ? 2 * i + 8 : I + i));
        const uint4 gv2 = *(const uint4*)(gu + t2 * 2 * I + (block ? 2 * i2 : i2));
        const uint4 uv2 = *(const uint4*)(gu + t2 * 2 * I + (block ? 2 * i2 + 8 : I + i2));
        *(uint4*)(out + t * I + i) = swiglu8(gv, uv);
        if (two) *(uint4*)(out + t2 * I + i2) = swiglu8(gv2, uv2);
    }
}

RB_EXPORT int rb_swiglu(const void* gu, void* out, int act_dtype, int T, int I, int block, cudaStream_t st) {
    if (T <= 0) return 0;
    if (block != 0 && (block != 8 || I % 8)) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    if (act_dtype == RB_BF16 && (I % 8) == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t total = (size_t)T * (I >> 3);
        int blocks = (int)((total + threads - 1) / threads);
        if (blocks > 148 * 16) blocks = 148 * 16;
        return rb_launch_pdl(swiglu_bf16x8_kernel, dim3(blocks), dim3(threads), 0, st, (const bf16*)gu, (bf16*)out, T, I, block);
    }
    const size_t total = (size_t)T * I;
    int blocks = (int)((total + threads - 1) / threads);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_dtype == RB_F32)
        swiglu_kernel<float><<<blocks, threads, 0, st>>>((const float*)gu, (float*)out, T, I, block);
    else
        swiglu_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)gu, (bf16*)out, T, I, block);
    return rb_launch_status();
}


// ---------------------------------------------------------------- a sublayer's output normed before it joins the stream
// For layers that norm a sublayer's output as well as its input: stream[r] += rmsnorm(delta[r]) * (offset_post + w_post),
// and, if asked, out[r] = rmsnorm(stream[r]) * (offset_next + w_next) for the sublayer that runs next: one kernel at
// every joint of such a layer.  float32 arithmetic; the row stays in shared memory between the two sums.
template <typename TA>
__global__ void postnorm_add_norm_kernel(float* __restrict__ stream, const TA* __restrict__ delta, const void* __restrict__ w_post,
                                         int wp_dtype, float eps_post, float offset_post, const void* __restrict__ w_next,
                                         int wn_dtype, float eps_next, float offset_next, TA* __restrict__ out, int H) {
    extern __shared__ float smem[];
    float* xrow = smem;          // H floats
    float* scratch = smem + H;   // 33 floats
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    float* s = stream + (size_t)row * H;
    const TA* d = delta + (size_t)row * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(d[i]);
        xrow[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rstd_d = 1.0f / sqrtf(ss / (float)H + eps_post);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = s[i] + xrow[i] * rstd_d * (offset_post + load_as_f32(w_post, wp_dtype, i));
        s[i] = x;
        xrow[i] = x;
        ss2 += x * x;
    }
    pdl_trigger_late();
    if (out == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float rstd = 1.0f / sqrtf(ss2 / (float)H + eps_next);
    TA* o = out + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f32<TA>(xrow[i] * rstd * (offset_next + load_as_f32(w_next, wn_dtype, i)));
}

RB_EXPORT int rb_postnorm_add_norm(float* stream, const void* delta, const void* w_post, int wp_dtype, float eps_post,
                                   float offset_post, const void* w_next, int wn_dtype, float eps_next, float offset_next,
                                   void* out, int act_dtype, int n_rows, int H, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    int threads = 128;
    while (threads < 1024 && threads * 8 < H) threads <<= 1;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(postnorm_add_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, st, stream, (const float*)delta,
                             w_post, wp_dtype, eps_post, offset_post, w_next, wn_dtype, eps_next, offset_next, (float*)out, H);
    return rb_launch_pdl(postnorm_add_norm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, st, stream, (const bf16*)delta, w_post,
                         wp_dtype, eps_post, offset_post, w_next, wn_dtype, eps_next, offset_next, (bf16*)out, H);
}

// ---------------------------------------------------------------- soft cap of the logits
// x <- cap * tanh(x / cap), in place, float32.
__global__ void softcap_kernel(float* __restrict__ x, float cap, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const float inv = 1.0f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

RB_EXPORT int rb_softcap(float* x, float cap, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    return rb_launch_pdl(softcap_kernel, dim3(blocks), dim3(256), 0, st, x, cap, total);
}

// ---------------------------------------------------------------- one-argument activations over rows
// out[r, c] = f(x[r, c]) for rows of `cols` elements with their own strides; in place when out == x.
// f by its number (rb_activate in common.cuh).  Arithmetic in float32; the input and the output each float32 or bfloat16.

template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ x, long long ldx, TO* __restrict__ out, long long ldo, int op,
                                  const void* __restrict__ bias, int bias_dtype, int rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)rows * cols;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / cols;
        const int c = (int)(e - r * cols);
        const float v = to_f32(x[r * ldx + c]);
        out[r * ldo + c] = from_f32<TO>(rb_activate(op, v, bias, bias_dtype, (size_t)c));
    }
}

RB_EXPORT int rb_activation(const void* x, long long ldx, int x_dtype, void* out, long long ldo, int out_dtype, int op,
                            const void* bias, int bias_dtype, int rows, int cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return 0;
    if (op < 0 || op > ACT_NEG_EXP_EXP) return (int)cudaErrorInvalidValue;
    const long long total = (long long)rows * cols;
    const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    if (x_dtype == RB_F32 && out_dtype == RB_F32)
        return rb_launch_pdl(activation_kernel<float, float>, dim3(blocks), dim3(256), 0, st, (const float*)x, ldx, (float*)out, ldo, op, bias, bias_dtype, rows, cols);
    if (x_dtype == RB_F32)
        return rb_launch_pdl(activation_kernel<float, bf16>, dim3(blocks), dim3(256), 0, st, (const float*)x, ldx, (bf16*)out, ldo, op, bias, bias_dtype, rows, cols);
    if (out_dtype == RB_F32)
        return rb_launch_pdl(activation_kernel<bf16, float>, dim3(blocks), dim3(256), 0, st, (const bf16*)x, ldx, (float*)out, ldo, op, bias, bias_dtype, rows, cols);
    return rb_launch_pdl(activation_kernel<bf16, bf16>, dim3(blocks), dim3(256), 0, st, (const bf16*)x, ldx, (bf16*)out, ldo, op, bias, bias_dtype, rows, cols);
}

// ---------------------------------------------------------------- several residual streams (hyper-connections)
// A token's residual is S streams x_0 .. x_(S-1), stored [T, S, H] in float32.  A sublayer reads one weighted sum of
// them and writes back into all of them:
//     read:   u = sum_s a[s] x_s;  out = u * rsqrt(mean(u^2) + eps) * (offset + w)
//     write:  x_t <- sum_s m[s, t] x_s + b[t] y   for all t at once from the old streams (m indexed [from, to]),
//             optionally followed by the read of the sublayer that runs next (its a, w), in the same kernel: the
//             row's new streams are still in registers.
// a, b, m are float32 (a null a reads the plain sum of the streams).  One CTA a token row; a thread holds the S values
// of its columns in registers, S <= HYPER_MAX_STREAMS.  With `rows` the read kernel takes only the listed rows.
#define HYPER_MAX_STREAMS 8

// VEC columns a thread and step (4 when H is a multiple of 4: 16-byte loads and stores of the streams; else 1).  Which
// columns a thread sums depends on H alone, so a row's sum of squares is added in one order whatever the step holds.
template <int VEC> __device__ __forceinline__ void hyper_load(const float* p, float (&v)[VEC]) {
    if constexpr (VEC == 4) { const float4 q = *reinterpret_cast<const float4*>(p); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    else v[0] = *p;
}
template <int VEC> __device__ __forceinline__ void hyper_load(const bf16* p, float (&v)[VEC]) {
    if constexpr (VEC == 4) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    } else v[0] = to_f32(*p);
}
template <int VEC> __device__ __forceinline__ void hyper_store(float* p, const float (&v)[VEC]) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <int VEC> __device__ __forceinline__ void hyper_store(bf16* p, const float (&v)[VEC]) {
    if constexpr (VEC == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 q;
        q.x = *reinterpret_cast<const unsigned*>(&lo);
        q.y = *reinterpret_cast<const unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = q;
    } else *p = __float2bfloat16_rn(v[0]);
}

// The normed rows from the sums a row left in shared memory.
template <typename TA, int VEC>
__device__ __forceinline__ void hyper_normed_rows(const float* u, float rstd, const void* w, int w_dtype, float offset,
                                                  TA* out_row, int H) {
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float o[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = u[i + e] * rstd * (offset + load_as_f32(w, w_dtype, (size_t)(i + e)));
        hyper_store<VEC>(out_row + i, o);
    }
}

template <typename TA, int S, int VEC>
__global__ void __launch_bounds__(256)
hyper_read_norm_kernel(const float* __restrict__ streams, const float* __restrict__ a, const int* __restrict__ rows,
                       const void* __restrict__ w, int w_dtype, float eps, float offset, TA* __restrict__ out, int H) {
    extern __shared__ __align__(16) float hyper_smem[];    // H floats, then 33 for the sum
    float* scratch = hyper_smem + ((H + 3) & ~3);
    float coef[S];                                         // parameters: nobody's output, read ahead of the wait
#pragma unroll
    for (int s = 0; s < S; ++s) coef[s] = a ? a[s] : 1.0f;
    pdl_wait();
    const size_t t = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    const float* x = streams + t * S * H;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float old[S][VEC];
#pragma unroll
        for (int s = 0; s < S; ++s) hyper_load<VEC>(x + (size_t)s * H + i, old[s]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s) u = fmaf(coef[s], old[s][e], u);
            hyper_smem[i + e] = u;
            ss = fmaf(u, u, ss);
        }
    }
    ss = block_sum(ss, scratch);
    pdl_trigger_late();
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    hyper_normed_rows<TA, VEC>(hyper_smem, rstd, w, w_dtype, offset, out + (size_t)blockIdx.x * H, H);
}

template <typename TA, typename TY, int S, int VEC>
__global__ void __launch_bounds__(256)
hyper_write_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ m,
                   const float* __restrict__ b, const float* __restrict__ a_next, const void* __restrict__ w_next,
                   int w_dtype, float eps, float offset, TA* __restrict__ out, int H) {
    extern __shared__ __align__(16) float hyper_smem[];
    float* scratch = hyper_smem + ((H + 3) & ~3);
    const size_t t = blockIdx.x;
    float* x = streams + t * S * H;
    float mix[S][S], bo[S], an[S];                         // parameters: nobody's output, read ahead of the wait
#pragma unroll
    for (int s = 0; s < S; ++s) {
        bo[s] = b[s];
        an[s] = out ? (a_next ? a_next[s] : 1.0f) : 0.f;
#pragma unroll
        for (int r = 0; r < S; ++r) mix[s][r] = m[s * S + r];
    }
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float old[S][VEC], yv[VEC], u[VEC];
#pragma unroll
        for (int s = 0; s < S; ++s) hyper_load<VEC>(x + (size_t)s * H + i, old[s]);
        hyper_load<VEC>(y + t * H + i, yv);
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = 0.f;
#pragma unroll
        for (int r = 0; r < S; ++r) {
            float v[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                v[e] = bo[r] * yv[e];
#pragma unroll
                for (int s = 0; s < S; ++s) v[e] = fmaf(mix[s][r], old[s][e], v[e]);
                u[e] = fmaf(an[r], v[e], u[e]);
            }
            hyper_store<VEC>(x + (size_t)r * H + i, v);
        }
        if (out) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                hyper_smem[i + e] = u[e];
                ss = fmaf(u[e], u[e], ss);
            }
        }
    }
    if (!out) return;
    ss = block_sum(ss, scratch);
    pdl_trigger_late();
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    hyper_normed_rows<TA, VEC>(hyper_smem, rstd, w_next, w_dtype, offset, out + t * H, H);
}

template <typename TA, int S>
static int hyper_read_launch(const float* streams, const float* a, const int* rows, const void* w, int w_dtype, float eps,
                             float offset, void* out, int n, int H, cudaStream_t st) {
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (H % 4 == 0 && (uintptr_t)streams % 16 == 0 && (uintptr_t)out % 16 == 0)
        return rb_launch_pdl(hyper_read_norm_kernel<TA, S, 4>, dim3(n), dim3(256), smem, st, streams, a, rows, w, w_dtype, eps,
                             offset, (TA*)out, H);
    return rb_launch_pdl(hyper_read_norm_kernel<TA, S, 1>, dim3(n), dim3(256), smem, st, streams, a, rows, w, w_dtype, eps, offset,
                         (TA*)out, H);
}

template <typename TA, typename TY, int S>
static int hyper_write_launch(float* streams, const void* y, const float* m, const float* b, const float* a_next,
                              const void* w_next, int w_dtype, float eps, float offset, void* out, int T, int H,
                              cudaStream_t st) {
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (H % 4 == 0 && (uintptr_t)streams % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0)
        return rb_launch_pdl(hyper_write_kernel<TA, TY, S, 4>, dim3(T), dim3(256), smem, st, streams, (const TY*)y, m, b, a_next,
                             w_next, w_dtype, eps, offset, (TA*)out, H);
    return rb_launch_pdl(hyper_write_kernel<TA, TY, S, 1>, dim3(T), dim3(256), smem, st, streams, (const TY*)y, m, b, a_next, w_next,
                         w_dtype, eps, offset, (TA*)out, H);
}

#define HYPER_BY_STREAMS(CALL)                                                   \
    switch (S) {                                                                 \
        case 1: return CALL(1); case 2: return CALL(2); case 3: return CALL(3); \
        case 4: return CALL(4); case 5: return CALL(5); case 6: return CALL(6); \
        case 7: return CALL(7); case 8: return CALL(8);                          \
        default: return (int)cudaErrorInvalidValue;                              \
    }

RB_EXPORT int rb_hyper_read_norm(const float* streams, const float* a, const int* rows, const void* w, int w_dtype, float eps,
                                 float offset, void* out, int act_dtype, int n, int S, int H, cudaStream_t st) {
    if (n <= 0) return 0;
    if ((size_t)(H + 36) * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (act_dtype == RB_F32) {
#define CALL(N) hyper_read_launch<float, N>(streams, a, rows, w, w_dtype, eps, offset, out, n, H, st)
        HYPER_BY_STREAMS(CALL)
#undef CALL
    }
#define CALL(N) hyper_read_launch<bf16, N>(streams, a, rows, w, w_dtype, eps, offset, out, n, H, st)
    HYPER_BY_STREAMS(CALL)
#undef CALL
}

RB_EXPORT int rb_hyper_write(float* streams, const void* y, int y_f32, const float* m, const float* b, const float* a_next,
                             const void* w_next, int w_dtype, float eps, float offset, void* out, int act_dtype, int T,
                             int S, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if ((size_t)(H + 36) * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (act_dtype == RB_F32) {                             // the 32-bit path: y is float32 as well
#define CALL(N) hyper_write_launch<float, float, N>(streams, y, m, b, a_next, w_next, w_dtype, eps, offset, out, T, H, st)
        HYPER_BY_STREAMS(CALL)
#undef CALL
    }
    if (y_f32) {
#define CALL(N) hyper_write_launch<bf16, float, N>(streams, y, m, b, a_next, w_next, w_dtype, eps, offset, out, T, H, st)
        HYPER_BY_STREAMS(CALL)
#undef CALL
    }
#define CALL(N) hyper_write_launch<bf16, bf16, N>(streams, y, m, b, a_next, w_next, w_dtype, eps, offset, out, T, H, st)
    HYPER_BY_STREAMS(CALL)
#undef CALL
}
