// What stands between an attention's projections and its paged attention kernel, and behind it, for attentions whose
// heads are prepared as a whole row rather than head by head; and the embedding with a table of token pairs.
//
//   attn_prep_kernel     one CTA a token.  From the projection row [q | k | v] (heads of `dim` key elements and `vdim`
//                        value elements): optional biases; optional RMS norm over the WHOLE q projection and over the
//                        whole k projection (a weight per element); optional rotation by position of the first `rot`
//                        elements of every q and k head, element 2i paired with 2i + 1; q heads written to a buffer of
//                        heads padded to D, k and v heads written into the pages (padded to D with zeros).  With
//                        v_off < 0 the values are the key projection as it came out of the product (before norm and
//                        rotation).  A run that reads another run's cache writes no keys and no values.
//   attn_gate_kernel     o[t, h, :] *= sigmoid(gate), one gate per head or one per value element.
//   embedding_pair_kernel, last_token_kernel
//                        stream[t] = scale * table[token] + pair_table[row], row = (prev * mul_prev + token * mul_cur) mod
//                        buckets, or row `buckets` for the first token of a sequence; the token before a step's first one
//                        is the request's kept token (an int per slot), which the second kernel renews after the step.
#include "common.cuh"

struct PrepArgs {
    const void* proj; int ld;
    int q_off, k_off, v_off;
    const void* q_bias; const void* k_bias; const void* v_bias; int bias_dtype;
    const void* q_norm; const void* k_norm; int norm_dtype; float eps;
    const float* cos_t; const float* sin_t; int rot;
    const int* pos; const int* tok_seg; const int* block_table; int bt_stride, page_size;
    void* kpool; void* vpool; void* q_out;
    int Hq, Hkv, dim, vdim, D, write_kv;
};

template <typename TA>
__global__ void __launch_bounds__(256)
attn_prep_kernel(const PrepArgs a) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
    const TA* row = (const TA*)a.proj + (size_t)t * a.ld;
    const int p = a.pos[t];
    const int nq = a.Hq * a.dim, nk = a.Hkv * a.dim;
    auto q_at = [&](int e) { return to_f32(row[a.q_off + e]) + (a.q_bias ? load_as_f32(a.q_bias, a.bias_dtype, e) : 0.f); };
    auto k_at = [&](int e) { return to_f32(row[a.k_off + e]) + (a.k_bias ? load_as_f32(a.k_bias, a.bias_dtype, e) : 0.f); };
    float rq = 1.f, rk = 1.f;
    if (a.q_norm) {
        float ss = 0.f;
        for (int e = tid; e < nq; e += nth) { const float v = q_at(e); ss = fmaf(v, v, ss); }
        ss = block_sum(ss, scratch);
        rq = 1.0f / sqrtf(ss / (float)nq + a.eps);
        if (a.write_kv) {
            ss = 0.f;
            for (int e = tid; e < nk; e += nth) { const float v = k_at(e); ss = fmaf(v, v, ss); }
            ss = block_sum(ss, scratch);
            rk = 1.0f / sqrtf(ss / (float)nk + a.eps);
        }
    }
    const int half = a.rot >> 1;
    const float* cs = a.cos_t + (size_t)p * half;
    const float* sn = a.sin_t + (size_t)p * half;
    const int pairs = a.D >> 1;                             // D is even
    // queries: pairs of neighbouring elements
    TA* qo = (TA*)a.q_out + (size_t)t * a.Hq * a.D;
    for (int e = tid; e < a.Hq * pairs; e += nth) {
        const int h = e / pairs, i = (e - h * pairs) * 2;
        float u = 0.f, v = 0.f;
        if (i < a.dim) {
            u = q_at(h * a.dim + i) * rq;
            if (a.q_norm) u *= load_as_f32(a.q_norm, a.norm_dtype, h * a.dim + i);
        }
        if (i + 1 < a.dim) {
            v = q_at(h * a.dim + i + 1) * rq;
            if (a.q_norm) v *= load_as_f32(a.q_norm, a.norm_dtype, h * a.dim + i + 1);
        }
        if (i < a.rot) {
            const float c = cs[i >> 1], s = sn[i >> 1];
            const float nu = u * c - v * s, nv = v * c + u * s;
            u = nu; v = nv;
        }
        qo[(size_t)h * a.D + i] = from_f32<TA>(u);
        qo[(size_t)h * a.D + i + 1] = from_f32<TA>(v);
    }
    if (!a.write_kv) return;
    const int page = a.block_table[(size_t)a.tok_seg[t] * a.bt_stride + p / a.page_size];
    if (page < 0) return;                                   // a padding row of a captured step: it has no page
    const size_t slot = ((size_t)page * a.Hkv * a.page_size + (size_t)(p % a.page_size)) * a.D;
    const size_t head_stride = (size_t)a.page_size * a.D;
    TA* kp = (TA*)a.kpool + slot;
    TA* vp = (TA*)a.vpool + slot;
    for (int e = tid; e < a.Hkv * pairs; e += nth) {
        const int h = e / pairs, i = (e - h * pairs) * 2;
        float u = 0.f, v = 0.f, u_raw = 0.f, v_raw = 0.f;
        if (i < a.dim) {
            u_raw = k_at(h * a.dim + i);
            u = u_raw * rk;
            if (a.k_norm) u *= load_as_f32(a.k_norm, a.norm_dtype, h * a.dim + i);
        }
        if (i + 1 < a.dim) {
            v_raw = k_at(h * a.dim + i + 1);
            v = v_raw * rk;
            if (a.k_norm) v *= load_as_f32(a.k_norm, a.norm_dtype, h * a.dim + i + 1);
        }
        if (i < a.rot) {
            const float c = cs[i >> 1], s = sn[i >> 1];
            const float nu = u * c - v * s, nv = v * c + u * s;
            u = nu; v = nv;
        }
        kp[h * head_stride + i] = from_f32<TA>(u);
        kp[h * head_stride + i + 1] = from_f32<TA>(v);
        if (a.v_off < 0) {                                  // the values are the keys as they were projected
            vp[h * head_stride + i] = from_f32<TA>(i < a.vdim ? u_raw : 0.f);
            vp[h * head_stride + i + 1] = from_f32<TA>(i + 1 < a.vdim ? v_raw : 0.f);
        }
    }
    if (a.v_off >= 0) {
        for (int e = tid; e < a.Hkv * a.D; e += nth) {
            const int h = e / a.D, i = e - h * a.D;
            float v = 0.f;
            if (i < a.vdim) {
                const int c = h * a.vdim + i;
                v = to_f32(row[a.v_off + c]) + (a.v_bias ? load_as_f32(a.v_bias, a.bias_dtype, c) : 0.f);
            }
            vp[h * head_stride + i] = from_f32<TA>(v);
        }
    }
}

// The bfloat16 form for sizes that are whole 16-byte pieces (dim, vdim, D, rot, the columns' offsets and the row stride
// multiples of 8 elements, every pointer aligned): a thread takes eight neighbouring elements of a head at a time, so
// the projections are read and the rows and pages written in 16-byte accesses.  Same arithmetic, element by element.
struct Vec8 { float v[8]; };
__device__ __forceinline__ Vec8 ld8(const bf16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    Vec8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); o.v[2 * j] = f.x; o.v[2 * j + 1] = f.y; }
    return o;
}
__device__ __forceinline__ void st8(bf16* p, const Vec8& x) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(x.v[2 * j], x.v[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__global__ void __launch_bounds__(256)
attn_prep_vec_kernel(const PrepArgs a) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
    const bf16* row = (const bf16*)a.proj + (size_t)t * a.ld;
    const int p = a.pos[t];
    const int nq = a.Hq * a.dim, nk = a.Hkv * a.dim;
    auto with_bias = [&](const bf16* src, const void* bias, int e) {      // eight projected elements from column e of their part
        Vec8 x = ld8(src + e);
        if (bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) x.v[j] += load_as_f32(bias, a.bias_dtype, e + j);
        }
        return x;
    };
    float rq = 1.f, rk = 1.f;
    if (a.q_norm) {
        float ss = 0.f;
        for (int e = tid * 8; e < nq; e += nth * 8) {
            const Vec8 x = with_bias(row + a.q_off, a.q_bias, e);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(x.v[j], x.v[j], ss);
        }
        ss = block_sum(ss, scratch);
        rq = 1.0f / sqrtf(ss / (float)nq + a.eps);
        if (a.write_kv) {
            ss = 0.f;
            for (int e = tid * 8; e < nk; e += nth * 8) {
                const Vec8 x = with_bias(row + a.k_off, a.k_bias, e);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(x.v[j], x.v[j], ss);
            }
            ss = block_sum(ss, scratch);
            rk = 1.0f / sqrtf(ss / (float)nk + a.eps);
        }
    }
    const int half = a.rot >> 1;
    const float* cs = a.cos_t + (size_t)p * half;
    const float* sn = a.sin_t + (size_t)p * half;
    auto finish = [&](Vec8& x, const void* w, float r, int e, int i) {    // norm weights, then the rotation of four pairs
        if (w) {
#pragma unroll
            for (int j = 0; j < 8; ++j) x.v[j] *= r * load_as_f32(w, a.norm_dtype, e + j);
        }
        if (i < a.rot) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float c = cs[(i >> 1) + j], s = sn[(i >> 1) + j];
                const float u = x.v[2 * j], v = x.v[2 * j + 1];
                x.v[2 * j] = u * c - v * s;
                x.v[2 * j + 1] = v * c + u * s;
            }
        }
    };
    const int chunks = a.D >> 3;
    Vec8 zero;
#pragma unroll
    for (int j = 0; j < 8; ++j) zero.v[j] = 0.f;
    bf16* qo = (bf16*)a.q_out + (size_t)t * a.Hq * a.D;
    for (int c = tid; c < a.Hq * chunks; c += nth) {
        const int h = c / chunks, i = (c - h * chunks) * 8;
        Vec8 x = zero;
        if (i < a.dim) {
            x = with_bias(row + a.q_off, a.q_bias, h * a.dim + i);
            finish(x, a.q_norm, rq, h * a.dim + i, i);
        }
        st8(qo + (size_t)h * a.D + i, x);
    }
    if (!a.write_kv) return;
    const int page = a.block_table[(size_t)a.tok_seg[t] * a.bt_stride + p / a.page_size];
    if (page < 0) return;
    const size_t slot = ((size_t)page * a.Hkv * a.page_size + (size_t)(p % a.page_size)) * a.D;
    const size_t head_stride = (size_t)a.page_size * a.D;
    bf16* kp = (bf16*)a.kpool + slot;
    bf16* vp = (bf16*)a.vpool + slot;
    for (int c = tid; c < a.Hkv * chunks; c += nth) {
        const int h = c / chunks, i = (c - h * chunks) * 8;
        Vec8 x = zero, raw = zero;
        if (i < a.dim) {
            x = raw = with_bias(row + a.k_off, a.k_bias, h * a.dim + i);
            finish(x, a.k_norm, rk, h * a.dim + i, i);
        }
        st8(kp + h * head_stride + i, x);
        if (a.v_off < 0) {
            st8(vp + h * head_stride + i, i < a.vdim ? raw : zero);
        } else {
            Vec8 v = zero;
            if (i < a.vdim) v = with_bias(row + a.v_off, a.v_bias, h * a.vdim + i);
            st8(vp + h * head_stride + i, v);
        }
    }
}

RB_EXPORT int rb_attn_prep(const void* proj, int ld, int q_off, int k_off, int v_off, const void* q_bias, const void* k_bias,
                           const void* v_bias, int bias_dtype, const void* q_norm, const void* k_norm, int norm_dtype, float eps,
                           const float* cos_t, const float* sin_t, int rot, const int* pos, const int* tok_seg,
                           const int* block_table, int bt_stride, int page_size, void* kpool, void* vpool, void* q_out,
                           int act_dtype, int T, int Hq, int Hkv, int dim, int vdim, int D, int write_kv, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D % 2 || dim > D || vdim > D || rot % 2 || rot > dim || (write_kv && v_off < 0 && vdim > dim)) return (int)cudaErrorInvalidValue;
    PrepArgs a;
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.q_bias = q_bias; a.k_bias = k_bias; a.v_bias = v_bias; a.bias_dtype = bias_dtype;
    a.q_norm = q_norm; a.k_norm = k_norm; a.norm_dtype = norm_dtype; a.eps = eps;
    a.cos_t = cos_t; a.sin_t = sin_t; a.rot = rot;
    a.pos = pos; a.tok_seg = tok_seg; a.block_table = block_table; a.bt_stride = bt_stride; a.page_size = page_size;
    a.kpool = kpool; a.vpool = vpool; a.q_out = q_out;
    a.Hq = Hq; a.Hkv = Hkv; a.dim = dim; a.vdim = vdim; a.D = D; a.write_kv = write_kv;
    auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = act_dtype == RB_BF16 && dim % 8 == 0 && vdim % 8 == 0 && D % 8 == 0 && rot % 8 == 0 && ld % 8 == 0 &&
                     q_off % 8 == 0 && k_off % 8 == 0 && (v_off < 0 || v_off % 8 == 0) && al(proj) && al(q_out) &&
                     al(kpool) && al(vpool);
    if (vec) return rb_launch_pdl(attn_prep_vec_kernel, dim3(T), dim3(256), 0, st, a);
    if (act_dtype == RB_F32) return rb_launch_pdl(attn_prep_kernel<float>, dim3(T), dim3(256), 0, st, a);
    return rb_launch_pdl(attn_prep_kernel<bf16>, dim3(T), dim3(256), 0, st, a);
}

// o: [T, H, D] in place; gate: rows of stride gate_ld, from column g_off: one per head (per_head) or [H, vdim].
template <typename TA>
__global__ void __launch_bounds__(256)
attn_gate_kernel(TA* __restrict__ o, const TA* __restrict__ gate, int gate_ld, int g_off, int per_head, int H, int vdim, int D,
                 size_t n) {
    pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / ((size_t)H * D);
        const int r = (int)(e - t * H * D), h = r / D, i = r - h * D;
        if (i >= vdim) continue;                            // the padding stays zero
        const float g = to_f32(gate[t * gate_ld + g_off + (per_head ? h : h * vdim + i)]);
        o[e] = from_f32<TA>(to_f32(o[e]) / (1.0f + expf(-g)));
    }
    pdl_trigger_late();
}

// The bfloat16 form for whole 16-byte pieces: eight neighbouring values of a head a thread and round.
__global__ void __launch_bounds__(256)
attn_gate_vec_kernel(bf16* __restrict__ o, const bf16* __restrict__ gate, int gate_ld, int g_off, int per_head, int H, int vdim,
                     int D, size_t n8) {
    pdl_wait();
    const int chunks = D >> 3;
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n8; c += (size_t)gridDim.x * blockDim.x) {
        const size_t t = c / ((size_t)H * chunks);
        const int r = (int)(c - t * H * chunks), h = r / chunks, i = (r - h * chunks) * 8;
        if (i >= vdim) continue;                            // the padding stays zero
        Vec8 x = ld8(o + c * 8);
        if (per_head) {
            const float g = 1.0f / (1.0f + expf(-to_f32(gate[t * gate_ld + g_off + h])));
#pragma unroll
            for (int j = 0; j < 8; ++j) x.v[j] *= g;
        } else {
            const Vec8 g = ld8(gate + t * gate_ld + g_off + h * vdim + i);
#pragma unroll
            for (int j = 0; j < 8; ++j) x.v[j] = x.v[j] / (1.0f + expf(-g.v[j]));
        }
        st8(o + c * 8, x);
    }
    pdl_trigger_late();
}

RB_EXPORT int rb_attn_gate(void* o, const void* gate, int gate_ld, int g_off, int per_head, int act_dtype, int T, int H,
                           int vdim, int D, cudaStream_t st) {
    const size_t n = (size_t)T * H * D;
    if (n == 0) return 0;
    if (act_dtype == RB_BF16 && D % 8 == 0 && vdim % 8 == 0 && ((uintptr_t)o & 15) == 0 &&
        (per_head || (gate_ld % 8 == 0 && g_off % 8 == 0 && ((uintptr_t)gate & 15) == 0))) {
        const size_t n8 = n / 8;
        const int vblocks = (int)((n8 + 255) / 256 < 8192 ? (n8 + 255) / 256 : 8192);
        return rb_launch_pdl(attn_gate_vec_kernel, dim3(vblocks), dim3(256), 0, st, (bf16*)o, (const bf16*)gate, gate_ld, g_off,
                             per_head, H, vdim, D, n8);
    }
    const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(attn_gate_kernel<float>, dim3(blocks), dim3(256), 0, st, (float*)o, (const float*)gate, gate_ld, g_off,
                             per_head, H, vdim, D, n);
    return rb_launch_pdl(attn_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, st, (bf16*)o, (const bf16*)gate, gate_ld, g_off,
                         per_head, H, vdim, D, n);
}

// ---------------------------------------------------------------- embedding with a table of token pairs
template <typename TW>
__global__ void __launch_bounds__(256)
embedding_pair_kernel(const TW* __restrict__ table, const TW* __restrict__ pairs, const int* __restrict__ tokens,
                      const int* __restrict__ pos, const int* __restrict__ tok_seg, const int* __restrict__ cu_q,
                      const int* __restrict__ seg_slot, const int* __restrict__ last_token, float* __restrict__ stream,
                      int H, int V, float scale, int buckets, long long mul_prev, long long mul_cur) {
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const bool bad = id < 0 || id >= V;
    int prow = buckets;                                     // the row of a token with nothing before it
    if (!bad && pos[t] > 0) {
        const int seg = tok_seg[t];
        const int prev = t > cu_q[seg] ? tokens[t - 1] : last_token[seg_slot[seg]];
        long long r = ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
        if (r < 0) r += buckets;
        prow = (int)r;
    }
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    const TW* pr = pairs + (size_t)prow * H;
    float* dst = stream + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        dst[i] = bad ? __int_as_float(0x7fc00000) : fmaf(to_f32(src[i]), scale, to_f32(pr[i]));
}

__global__ void last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ cu_q,
                                  const int* __restrict__ seg_slot, int* __restrict__ last_token, int segments) {
    pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < segments) last_token[seg_slot[s]] = tokens[cu_q[s + 1] - 1];
}

RB_EXPORT int rb_embedding_pair(const void* table, const void* pairs, int table_dtype, const int* tokens, const int* pos,
                                const int* tok_seg, const int* cu_q, const int* seg_slot, const int* last_token,
                                float* stream, int T, int H, int V, float scale, int buckets, long long mul_prev,
                                long long mul_cur, cudaStream_t st) {
    if (T <= 0) return 0;
    if (buckets <= 0) return (int)cudaErrorInvalidValue;
    if (table_dtype == RB_F32)
        return rb_launch_pdl(embedding_pair_kernel<float>, dim3(T), dim3(256), 0, st, (const float*)table, (const float*)pairs,
                             tokens, pos, tok_seg, cu_q, seg_slot, last_token, stream, H, V, scale, buckets, mul_prev, mul_cur);
    return rb_launch_pdl(embedding_pair_kernel<bf16>, dim3(T), dim3(256), 0, st, (const bf16*)table, (const bf16*)pairs,
                         tokens, pos, tok_seg, cu_q, seg_slot, last_token, stream, H, V, scale, buckets, mul_prev, mul_cur);
}

RB_EXPORT int rb_last_token(const int* tokens, const int* cu_q, const int* seg_slot, int* last_token, int segments,
                            cudaStream_t st) {
    if (segments <= 0) return 0;
    return rb_launch_pdl(last_token_kernel, dim3((segments + 127) / 128), dim3(128), 0, st, tokens, cu_q, seg_slot, last_token,
                         segments);
}
