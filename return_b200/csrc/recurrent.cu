// Kernels of the mixers that carry a matrix state per head instead of cached keys: linear attention with a
// fixed decay (retention), the gated delta rule with a decay per key channel, and the matrix memory with
// exponential gates; plus the elementwise steps around them.
//
// A head's state S is a [D, V] matrix in float32 that is read out as o = S^T q.  One token's update is
//     fixed decay:     S <- a S + k v^T                                   o = S^T q
//     delta rule:      S <- g * S (row i by g_i);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//     delta rule, one decay a head: the same with a scalar g per token and head
//     matrix memory:   m' = max(f + m, i);  a = exp(f + m - m'),  b = exp(i - m');
//                      S <- a S + b k v^T;  n <- a n + b k;  o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//     bonus rule:      o = (S + diag(u) k v^T)^T q;  S <- g * S (row i by g_i) + k v^T: the token's own pair is read with
//                      a weight u per head and key row before the state takes it in (time mixing with a decay per token
//                      and key row)
//     state space:     S <- a S + dt k v^T;  o = S^T q + d v, with a decay a and a step dt per token and head and a
//                      skip weight d per head (k and q are the input and output maps of a group of heads)
// All of it is float32 whatever the activation type is.  The scan kernel walks the tokens of a segment in order,
// one after the other, for prompts and single tokens alike: a token's result therefore does not depend on how a
// prompt was cut into steps or on what else is in the batch (the sums have one fixed order).
//
// Thread layout of the scan: a CTA of 256 threads owns 32 value columns of one head of one segment.  R = 8
// neighbouring lanes share a column and split its D rows between them (lane r holds rows r, r + 8, ...), so a
// column's dot products end with three shuffles.  (The kernel is written for any R; 16 and 32 lanes a column, which
// spread a head of a long prompt over two and four times as many SMs, were measured slower: 0.64 and 0.76 ms against
// 0.47 for 2,048 tokens of 16 heads, because the longer chain of shuffles is what a token waits for.)  The state of a
// request lives in its slot in the same order, [head][row / 8][column][row % 8], which makes a warp's loads and
// stores of it whole 128-byte lines.  A twin of the kernel for steps of single tokens (nothing staged, every thread
// loading its rows of q and k itself) was measured too: 26 / 20 / 10 us against 7 / 15 / 11 for 8 requests of 16
// heads (fixed decay / matrix memory / delta rule), 171 / 135 / 65 against 42 / 99 / 75 for 64; not kept.
#include "common.cuh"

#define SCAN_THREADS 256
#define SCAN_TC 8             // tokens staged in shared memory at a time

#define MODE_DECAY 0
#define MODE_MEMORY 1
#define MODE_DELTA 2
#define MODE_BONUS 3
#define MODE_SSM 4
#define MODE_DELTA_HEAD 5

struct ScanArgs {
    const void* q; const void* k; const void* v;        // (t, head, i) at base + t * ld + head * dim + i
    int q_ld, k_ld, v_ld;
    int q_f32, k_f32, v_f32;                            // 1: float32, 0: bfloat16
    const float* gate_a;      // decay: [H] decays; memory: [T, 2H] gate pre-activations (input, forget); delta and bonus:
                              // [T, H*D] row decays; state space: [T, H] decays
    const float* gate_b;      // memory: [2H] gate biases; delta: [T, H] beta; state space: [T, H] steps
                              // delta with one decay a head: gate_a [T, H] decays, gate_b [T, H] beta
    const float* extra;       // bonus: [H, D] weights of the token's own pair; state space: [H] skip weights
    float cap, q_scale;
    float* state;             // [slots, state_stride]
    long long state_stride;
    int s_off, n_off, m_off;  // where S, n and m start inside a slot's row
    int f_off;                // matrix memory: where the sum of the segment's log forget gates goes per head, or -1
    const int* cu_q; const int* seg_slot;
    float* out;               // [T, H*V]
    int H, G, D, V;
};

__device__ __forceinline__ float ld_elem(const void* p, int f32, size_t i) {
    return f32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

// Sum over the R neighbouring lanes that share a column (R = 8, 16 or 32), in a fixed order.
template <int R>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoid_f(float x) { return x < 0.f ? x - log1pf(expf(x)) : -log1pf(expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int MODE, int NR, int R>
__global__ void __launch_bounds__(SCAN_THREADS, NR <= 16 ? 2 : 1)
linear_scan_kernel(const ScanArgs a) {
    constexpr int DP = NR * R;                         // rows the threads of a column can hold
    constexpr int SCAN_COLS = SCAN_THREADS / R;        // value columns of a CTA
    // a token's q, k (and row decays) as [row % R][row / R], each run of NR padded by four floats: a thread reads its
    // NR values as 16-byte pieces, and the eight runs that one such request covers fall on different banks
    constexpr int RS = NR + 4, DS = R * RS;
    constexpr int PER = SCAN_TC * DP / SCAN_THREADS;   // q (and k) elements of a chunk that a thread brings in
    constexpr bool ROW_DECAY = MODE == MODE_DELTA || MODE == MODE_BONUS;     // a decay per token, head and key row
    static_assert(SCAN_TC * SCAN_COLS <= SCAN_THREADS && (SCAN_TC * DP) % SCAN_THREADS == 0, "staging by all threads");
    pdl_wait();
    __shared__ __align__(16) float sq[SCAN_TC][DS];
    __shared__ __align__(16) float sk[SCAN_TC][DS];
    __shared__ __align__(16) float sg[ROW_DECAY ? SCAN_TC : 1][DS];
    __shared__ float sv[SCAN_TC][SCAN_COLS];
    __shared__ float sa[SCAN_TC], sb[SCAN_TC];
    const int seg = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * SCAN_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane % R, jj = warp * (32 / R) + lane / R, j = j0 + jj;
    const int H = a.H, D = a.D, V = a.V;
    const int kvh = h / (H / a.G);
    const int nrd = (D + 7) >> 3;                      // row groups that exist
    const int t0 = a.cu_q[seg], t1 = a.cu_q[seg + 1];
    float* st = a.state + (long long)a.seg_slot[seg] * a.state_stride;
    float* Sg = st + a.s_off + (size_t)h * nrd * 8 * V;
    const bool col = j < V;

    float S[NR], n[MODE == MODE_MEMORY ? NR : 1];
    float m = 0.f, forgot = 0.f;
#pragma unroll
    for (int ii = 0; ii < NR; ++ii) {
        const int row = r + R * ii;                    // rows beyond the padded key size do not exist: they stay zero
        S[ii] = (col && row < nrd * 8) ? Sg[((size_t)(row >> 3) * V + j) * 8 + (row & 7)] : 0.f;
    }
    if (MODE == MODE_MEMORY) {
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int row = r + R * ii;
            n[ii] = row < nrd * 8 ? st[a.n_off + (size_t)h * nrd * 8 + row] : 0.f;
        }
        m = st[a.m_off + h];
    }
    const float decay = MODE == MODE_DECAY ? a.gate_a[h] : 0.f;
    const float skip = MODE == MODE_SSM ? a.extra[h] : 0.f;
    float bonus[MODE == MODE_BONUS ? NR : 1];
    if (MODE == MODE_BONUS) {
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int row = r + R * ii;
            bonus[ii] = row < D ? a.extra[(size_t)h * D + row] : 0.f;
        }
    }
    const float bias_i = MODE == MODE_MEMORY ? a.gate_b[h] : 0.f, bias_f = MODE == MODE_MEMORY ? a.gate_b[H + h] : 0.f;

    // A chunk of up to SCAN_TC tokens comes from global memory into registers while the chunk before it is worked on,
    // and goes to shared memory when that is done.  The registers hold the loaded bits untouched: a conversion or a
    // product right behind a load would make the warp wait for it there, before the arithmetic it is meant to hide
    // behind.  Converting, scaling and the gates' transcendental functions happen on the way to shared memory.
    uint32_t rq[PER], rk[PER], rv = 0u;
    float rg[ROW_DECAY ? PER : 1], ra = 0.f, rb = 0.f;
    auto raw = [](const void* p, int f32, size_t i) -> uint32_t {
        return f32 ? ((const uint32_t*)p)[i] : (uint32_t)((const unsigned short*)p)[i];
    };
    auto cooked = [](uint32_t bits, int f32) -> float { return __uint_as_float(f32 ? bits : bits << 16); };
    auto fetch = [&](int tc) {
        const int nt = min(SCAN_TC, t1 - tc);
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int e = tid + u * SCAN_THREADS, tt = e / DP, i = e - tt * DP;
            const size_t t = (size_t)(tc + tt);
            const bool live = tt < nt && i < D;
            rq[u] = live ? raw(a.q, a.q_f32, t * a.q_ld + (size_t)kvh * D + i) : 0u;
            rk[u] = live ? raw(a.k, a.k_f32, t * a.k_ld + (size_t)kvh * D + i) : 0u;
            if (ROW_DECAY) rg[u] = live ? a.gate_a[(t * H + h) * D + i] : 1.f;
        }
        if (tid < SCAN_TC * SCAN_COLS) {
            const int tt = tid / SCAN_COLS, c = tid - tt * SCAN_COLS;
            rv = (tt < nt && j0 + c < V) ? raw(a.v, a.v_f32, (size_t)(tc + tt) * a.v_ld + (size_t)h * V + j0 + c) : 0u;
        }
        if (tid < nt) {
            const size_t t = (size_t)(tc + tid);
            if (MODE == MODE_MEMORY) {
                ra = a.gate_a[t * 2 * H + h];
                rb = a.gate_a[t * 2 * H + H + h];
            } else if (MODE == MODE_DELTA) {
                rb = a.gate_b[t * H + h];
            } else if (MODE == MODE_SSM || MODE == MODE_DELTA_HEAD) {
                ra = a.gate_a[t * H + h];
                rb = a.gate_b[t * H + h];
            }
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int e = tid + u * SCAN_THREADS, tt = e / DP, i = e - tt * DP;
            const int at = (i % R) * RS + i / R;
            sq[tt][at] = cooked(rq[u], a.q_f32) * a.q_scale;
            sk[tt][at] = cooked(rk[u], a.k_f32);
            if (ROW_DECAY) sg[tt][at] = rg[u];
        }
        if (tid < SCAN_TC * SCAN_COLS) sv[tid / SCAN_COLS][tid % SCAN_COLS] = cooked(rv, a.v_f32);
        if (tid < SCAN_TC) {
            if (MODE == MODE_MEMORY) {
                sa[tid] = a.cap * tanhf((ra + bias_i) / a.cap);
                sb[tid] = logsigmoid_f(a.cap * tanhf((rb + bias_f) / a.cap));
            } else {
                sa[tid] = ra;
                sb[tid] = rb;
            }
        }
    };
    // One token's update of the state.  A column's sums over its rows run as four partial sums per thread, added
    // pairwise; the sum over the eight threads of a column (three shuffles) can be left to the end of the chunk, where
    // the shuffles of all its tokens go out back to back.  The delta rule needs one such sum inside the token all the
    // same (its write depends on what the state holds for the key).
    float op[SCAN_TC], np[MODE == MODE_MEMORY ? SCAN_TC : 1], floor_[MODE == MODE_MEMORY ? SCAN_TC : 1];
    auto token = [&](int tt) {
        const float vj = sv[tt][jj];
        float kr[NR], qr[NR];
#pragma unroll
        for (int i4 = 0; i4 < NR; i4 += 4) {
            *(float4*)&kr[i4] = *(const float4*)&sk[tt][r * RS + i4];
            *(float4*)&qr[i4] = *(const float4*)&sq[tt][r * RS + i4];
        }
        float o4[4] = {0.f, 0.f, 0.f, 0.f};
        if (MODE == MODE_DECAY) {
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) {
                S[ii] = fmaf(decay, S[ii], kr[ii] * vj);
                o4[ii & 3] = fmaf(S[ii], qr[ii], o4[ii & 3]);
            }
        } else if (MODE == MODE_MEMORY) {
            const float lf = sb[tt], li = sa[tt];
            const float m_new = fmaxf(lf + m, li);
            const float fa = expf(lf + m - m_new), fb = expf(li - m_new);
            m = m_new;
            forgot += lf;
            floor_[tt] = expf(-m_new);
            float n4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) {
                const float bk = fb * kr[ii];
                S[ii] = fmaf(fa, S[ii], bk * vj);
                n[ii] = fmaf(fa, n[ii], bk);
                o4[ii & 3] = fmaf(S[ii], qr[ii], o4[ii & 3]);
                n4[ii & 3] = fmaf(n[ii], qr[ii], n4[ii & 3]);
            }
            np[tt] = (n4[0] + n4[1]) + (n4[2] + n4[3]);
        } else if (MODE == MODE_BONUS) {
            float gr[NR];
#pragma unroll
            for (int i4 = 0; i4 < NR; i4 += 4) *(float4*)&gr[i4] = *(const float4*)&sg[tt][r * RS + i4];
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) {
                const float kv = kr[ii] * vj;
                o4[ii & 3] = fmaf(fmaf(bonus[ii], kv, S[ii]), qr[ii], o4[ii & 3]);
                S[ii] = fmaf(gr[ii], S[ii], kv);
            }
        } else if (MODE == MODE_SSM) {
            const float fa = sa[tt], vdt = sb[tt] * vj;
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) {
                S[ii] = fmaf(fa, S[ii], kr[ii] * vdt);
                o4[ii & 3] = fmaf(S[ii], qr[ii], o4[ii & 3]);
            }
        } else {
            if (MODE == MODE_DELTA_HEAD) {
                const float g1 = sa[tt];
#pragma unroll
                for (int ii = 0; ii < NR; ++ii) S[ii] *= g1;
            } else {
#pragma unroll
                for (int i4 = 0; i4 < NR; i4 += 4) {
                    const float4 g4 = *(const float4*)&sg[tt][r * RS + i4];
                    S[i4] *= g4.x; S[i4 + 1] *= g4.y; S[i4 + 2] *= g4.z; S[i4 + 3] *= g4.w;
                }
            }
            float k4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) k4[ii & 3] = fmaf(S[ii], kr[ii], k4[ii & 3]);
            const float kv = lanes_sum<R>((k4[0] + k4[1]) + (k4[2] + k4[3]));
            const float u = sb[tt] * (vj - kv);
#pragma unroll
            for (int ii = 0; ii < NR; ++ii) {
                S[ii] = fmaf(kr[ii], u, S[ii]);
                o4[ii & 3] = fmaf(S[ii], qr[ii], o4[ii & 3]);
            }
        }
        op[tt] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    };
    auto finish = [&](int tt, int t) {
        float o = lanes_sum<R>(op[tt]);
        if (MODE == MODE_MEMORY) {
            const float nq = lanes_sum<R>(np[tt]);
            o = o / (fmaxf(fabsf(nq), floor_[tt]) + 1e-6f);
        }
        if (MODE == MODE_SSM) o = fmaf(skip, sv[tt][jj], o);
        if (r == 0 && col) a.out[((size_t)t * H + h) * V + j] = o;
    };

    if (t0 < t1) fetch(t0);
    for (int tc = t0; tc < t1; tc += SCAN_TC) {
        const int nt = min(SCAN_TC, t1 - tc);
        __syncthreads();                               // the chunk before this one has been used
        stash();
        __syncthreads();
        if (tc + SCAN_TC < t1) fetch(tc + SCAN_TC);    // in flight while this chunk is worked on
        if (nt == SCAN_TC) {
            if (MODE == MODE_DECAY) {                  // measured: 0.47 ms against 0.51 for 2,048 tokens of 16 heads
#pragma unroll
                for (int tt = 0; tt < SCAN_TC; ++tt) { token(tt); finish(tt, tc + tt); }
            } else {                                   // 0.94 against 0.97 (matrix memory), 0.86 against 0.88 (delta rule)
#pragma unroll
                for (int tt = 0; tt < SCAN_TC; ++tt) token(tt);
#pragma unroll
                for (int tt = 0; tt < SCAN_TC; ++tt) finish(tt, tc + tt);
            }
        } else {
#pragma unroll
            for (int tt = 0; tt < SCAN_TC; ++tt)
                if (tt < nt) token(tt);
#pragma unroll
            for (int tt = 0; tt < SCAN_TC; ++tt)
                if (tt < nt) finish(tt, tc + tt);
        }
    }
    pdl_trigger_late();
    if (col) {
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int row = r + R * ii;
            if (row < nrd * 8) Sg[((size_t)(row >> 3) * V + j) * 8 + (row & 7)] = S[ii];
        }
    }
    if (MODE == MODE_MEMORY && blockIdx.x == 0 && warp == 0 && lane < R) {
#pragma unroll
        for (int ii = 0; ii < NR; ++ii) {
            const int row = r + R * ii;
            if (row < nrd * 8) st[a.n_off + (size_t)h * nrd * 8 + row] = n[ii];
        }
        if (lane == 0) {
            st[a.m_off + h] = m;
            if (a.f_off >= 0) st[a.f_off + h] = forgot;
        }
    }
}

template <int MODE>
static int launch_scan(const ScanArgs& a, int segments, cudaStream_t st) {
    if (segments <= 0) return 0;
    if (a.D <= 0 || a.D > 256 || a.V <= 0 || a.G <= 0 || a.H % a.G) return (int)cudaErrorInvalidValue;
    constexpr int R = 8;
    dim3 grid((a.V + SCAN_THREADS / R - 1) / (SCAN_THREADS / R), a.H, segments);
    // rows a thread holds: the key size over the lanes of a column, rounded up to 4, 8, 16 or 32
    if (a.D <= 32) return rb_launch_pdl(linear_scan_kernel<MODE, 4, R>, grid, dim3(SCAN_THREADS), 0, st, a);
    if (a.D <= 64) return rb_launch_pdl(linear_scan_kernel<MODE, 8, R>, grid, dim3(SCAN_THREADS), 0, st, a);
    if (a.D <= 128) return rb_launch_pdl(linear_scan_kernel<MODE, 16, R>, grid, dim3(SCAN_THREADS), 0, st, a);
    return rb_launch_pdl(linear_scan_kernel<MODE, 32, R>, grid, dim3(SCAN_THREADS), 0, st, a);
}

// mode: 0 fixed decay, 1 matrix memory, 2 delta rule, 3 bonus rule, 4 state space.  The arguments are those of
// ScanArgs, in its order.
RB_EXPORT int rb_linear_scan(int mode, const void* q, const void* k, const void* v, int q_ld, int k_ld, int v_ld,
                             int q_f32, int k_f32, int v_f32, const float* gate_a, const float* gate_b,
                             const float* extra, float cap,
                             float q_scale, float* state, long long state_stride, int s_off, int n_off, int m_off,
                             int f_off, const int* cu_q, const int* seg_slot, float* out, int H, int G, int D, int V,
                             int segments, cudaStream_t st) {
    ScanArgs a;
    a.q = q; a.k = k; a.v = v; a.q_ld = q_ld; a.k_ld = k_ld; a.v_ld = v_ld;
    a.q_f32 = q_f32; a.k_f32 = k_f32; a.v_f32 = v_f32;
    a.gate_a = gate_a; a.gate_b = gate_b; a.extra = extra; a.cap = cap; a.q_scale = q_scale;
    a.state = state; a.state_stride = state_stride; a.s_off = s_off; a.n_off = n_off; a.m_off = m_off; a.f_off = f_off;
    a.cu_q = cu_q; a.seg_slot = seg_slot; a.out = out; a.H = H; a.G = G; a.D = D; a.V = V;
    if (mode == MODE_DECAY) return launch_scan<MODE_DECAY>(a, segments, st);
    if (mode == MODE_MEMORY) return launch_scan<MODE_MEMORY>(a, segments, st);
    if (mode == MODE_DELTA) return launch_scan<MODE_DELTA>(a, segments, st);
    if (mode == MODE_BONUS) return extra ? launch_scan<MODE_BONUS>(a, segments, st) : (int)cudaErrorInvalidValue;
    if (mode == MODE_SSM) return extra && gate_b ? launch_scan<MODE_SSM>(a, segments, st) : (int)cudaErrorInvalidValue;
    if (mode == MODE_DELTA_HEAD) return gate_b ? launch_scan<MODE_DELTA_HEAD>(a, segments, st) : (int)cudaErrorInvalidValue;
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------- a long segment cut into pieces that are scanned side by side
// With a fixed decay the state after a piece of n tokens is decay^n * (state before it) + (what the piece alone leaves
// behind, scanned from zero).  So the pieces of a long segment can be scanned from zero all at once; this kernel then
// walks a segment's pieces in order, puts the state each piece starts from where the piece's own result was
// (pieces[p] <- carry; carry <- decay^n carry + pieces[p]) and leaves the last carry in the request's slot; a second
// scan of the pieces from those states gives the outputs.  One thread an element of the state.
__global__ void scan_pieces_combine_kernel(float* __restrict__ pieces, long long piece_stride, float* __restrict__ state,
                                           long long state_stride, int s_off, const float* __restrict__ decay,
                                           const int* __restrict__ cu_piece, const int* __restrict__ seg_first,
                                           const int* __restrict__ seg_slot, int per_head, int total) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const float log_decay = logf(decay[e / per_head]);
    float* home = state + (long long)seg_slot[seg] * state_stride + s_off + e;
    float carry = *home;
    for (int p = seg_first[seg]; p < seg_first[seg + 1]; ++p) {
        float* at = pieces + (long long)p * piece_stride + e;
        const float left = *at;
        *at = carry;
        carry = fmaf(expf((float)(cu_piece[p + 1] - cu_piece[p]) * log_decay), carry, left);
    }
    *home = carry;
}

RB_EXPORT int rb_scan_pieces_combine(float* pieces, long long piece_stride, float* state, long long state_stride, int s_off,
                                     const float* decay, const int* cu_piece, const int* seg_first, const int* seg_slot,
                                     int per_head, int total, int segments, cudaStream_t st) {
    if (segments <= 0 || total <= 0) return 0;
    dim3 grid((total + 255) / 256, segments);
    return rb_launch_pdl(scan_pieces_combine_kernel, grid, dim3(256), 0, st, pieces, piece_stride, state, state_stride, s_off,
                         decay, cu_piece, seg_first, seg_slot, per_head, total);
}

// The same for decays that differ from token to token: per head (the state-space scan) or per head and key row (the
// scan with a bonus).  A piece's transition is then the product of its tokens' decays, which the first kernel leaves as
// a sum of logarithms per piece (a decay of zero gives minus infinity and a factor of zero); the second is the walk above with that factor.  An element e of a head's matrix
// belongs to key row (e / (8 V)) * 8 + e % 8 of the layout [row / 8][column][row % 8].
__global__ void piece_decay_sums_kernel(const float* __restrict__ decay, int n, const int* __restrict__ cu_piece,
                                        float* __restrict__ sums) {
    // 64 columns by 8 runs of tokens (token t of the piece goes to run t % 8); the runs are added in their order
    __shared__ float part[8][64];
    pdl_wait();
    const int p = blockIdx.y, i = blockIdx.x * 64 + threadIdx.x;
    float acc = 0.f;
    if (i < n)
        for (int t = cu_piece[p] + threadIdx.y; t < cu_piece[p + 1]; t += 8) acc += logf(decay[(size_t)t * n + i]);
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && i < n) {
#pragma unroll
        for (int y = 1; y < 8; ++y) acc += part[y][threadIdx.x];
        sums[(size_t)p * n + i] = acc;
    }
}

__global__ void scan_pieces_combine_sums_kernel(float* __restrict__ pieces, long long piece_stride, float* __restrict__ state,
                                                long long state_stride, int s_off, const float* __restrict__ sums, int n,
                                                int by_row, int D, int V, const int* __restrict__ seg_first,
                                                const int* __restrict__ seg_slot, int per_head, int total) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int h = e / per_head, rem = e - h * per_head;
    const int row = (rem / (8 * V)) * 8 + (rem & 7);
    float* home = state + (long long)seg_slot[seg] * state_stride + s_off + e;
    if (by_row && row >= D) return;                     // a padding row: it holds zero and stays zero
    const int col = by_row ? h * D + row : h;
    float carry = *home;
    for (int p = seg_first[seg]; p < seg_first[seg + 1]; ++p) {
        float* at = pieces + (long long)p * piece_stride + e;
        const float left = *at;
        *at = carry;
        carry = fmaf(expf(sums[(size_t)p * n + col]), carry, left);
    }
    *home = carry;
}

// decay: float32 [T, n] (n = heads, or heads * D with by_row); sums: float32 scratch [pieces, n]
RB_EXPORT int rb_scan_pieces_combine_sums(float* pieces, long long piece_stride, float* state, long long state_stride, int s_off,
                                          const float* decay, float* sums, int n, int by_row, int D, int V,
                                          const int* cu_piece, const int* seg_first, const int* seg_slot, int per_head,
                                          int total, int n_pieces, int segments, cudaStream_t st) {
    if (segments <= 0 || total <= 0 || n_pieces <= 0) return 0;
    if (per_head % (8 * V) || n <= 0) return (int)cudaErrorInvalidValue;
    int rc = rb_launch_pdl(piece_decay_sums_kernel, dim3((n + 63) / 64, n_pieces), dim3(64, 8), 0, st, decay, n, cu_piece, sums);
    if (rc) return rc;
    dim3 grid((total + 255) / 256, segments);
    return rb_launch_pdl(scan_pieces_combine_sums_kernel, grid, dim3(256), 0, st, pieces, piece_stride, state, state_stride,
                         s_off, (const float*)sums, n, by_row, D, V, seg_first, seg_slot, per_head, total);
}

// The same for the matrix memory.  A piece scanned from nothing (S = 0, n = 0, m = -infinity) leaves S', n', its own
// running maximum m' and F, the sum of its log forget gates; behind a state (S0, n0, m0) the piece ends in
//     m = max(F + m0, m'),   S = e^(F + m0 - m) S0 + e^(m' - m) S',   n likewise.
// The first kernel walks S and n (one thread an element; it reads every piece's m' and F and writes neither), the
// second, launched behind it, walks the maxima (one thread a head).
__global__ void memory_pieces_combine_kernel(float* __restrict__ pieces, long long piece_stride, float* __restrict__ state,
                                             long long state_stride, int s_off, int n_off, int m_off, int f_off,
                                             const int* __restrict__ seg_first, const int* __restrict__ seg_slot,
                                             int per_head_s, int per_head_n, int total_s, int total) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int h = e < total_s ? e / per_head_s : (e - total_s) / per_head_n;
    const int at = e < total_s ? s_off + e : n_off + (e - total_s);
    float* home = state + (long long)seg_slot[seg] * state_stride;
    float carry = home[at], m = home[m_off + h];
    for (int p = seg_first[seg]; p < seg_first[seg + 1]; ++p) {
        float* row = pieces + (long long)p * piece_stride;
        const float left = row[at], m_piece = row[m_off + h], forgot = row[f_off + h];
        row[at] = carry;
        const float m_new = fmaxf(forgot + m, m_piece);
        carry = fmaf(expf(forgot + m - m_new), carry, expf(m_piece - m_new) * left);
        m = m_new;
    }
    home[at] = carry;
}

__global__ void memory_pieces_maxima_kernel(float* __restrict__ pieces, long long piece_stride, float* __restrict__ state,
                                            long long state_stride, int m_off, int f_off, const int* __restrict__ seg_first,
                                            const int* __restrict__ seg_slot, int H) {
    pdl_wait();
    const int seg = blockIdx.y, h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= H) return;
    float* home = state + (long long)seg_slot[seg] * state_stride;
    float m = home[m_off + h];
    for (int p = seg_first[seg]; p < seg_first[seg + 1]; ++p) {
        float* row = pieces + (long long)p * piece_stride;
        const float m_piece = row[m_off + h], forgot = row[f_off + h];
        row[m_off + h] = m;
        m = fmaxf(forgot + m, m_piece);
    }
    home[m_off + h] = m;
}

RB_EXPORT int rb_memory_pieces_combine(float* pieces, long long piece_stride, float* state, long long state_stride, int s_off,
                                       int n_off, int m_off, int f_off, const int* seg_first, const int* seg_slot,
                                       int per_head_s, int per_head_n, int H, int segments, cudaStream_t st) {
    if (segments <= 0) return 0;
    const int total_s = H * per_head_s, total = total_s + H * per_head_n;
    int rc = rb_launch_pdl(memory_pieces_combine_kernel, dim3((total + 255) / 256, segments), dim3(256), 0, st, pieces,
                           piece_stride, state, state_stride, s_off, n_off, m_off, f_off, seg_first, seg_slot, per_head_s,
                           per_head_n, total_s, total);
    if (rc) return rc;
    return rb_launch_pdl(memory_pieces_maxima_kernel, dim3((H + 63) / 64, segments), dim3(64), 0, st, pieces, piece_stride,
                         state, state_stride, m_off, f_off, seg_first, seg_slot, H);
}

// ---------------------------------------------------------------- rotation of q and k into float32
// x: two runs of `heads` heads of size D inside rows of a projection buffer (q at q_off, k at k_off).  The first
// `rot` elements of a head turn by the angle of the token's position (tables cos, sin [positions, rot/2]), element
// i paired with i + rot/2; k is then multiplied by k_scale.  Results go to q32, k32 [T, heads, D].
template <typename TA>
__global__ void rotary_to_f32_kernel(const TA* __restrict__ x, int ld, int q_off, int k_off,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                     const int* __restrict__ pos, float* __restrict__ q32, float* __restrict__ k32,
                                     int heads, int D, float q_scale, float k_scale) {
    pdl_wait();
    const int t = blockIdx.x, hh = blockIdx.y;           // hh < heads: q, else k
    const bool is_k = hh >= heads;
    const int h = is_k ? hh - heads : hh;
    const TA* src = x + (size_t)t * ld + (is_k ? k_off : q_off) + (size_t)h * D;
    float* dst = (is_k ? k32 : q32) + ((size_t)t * heads + h) * D;
    const float scale = is_k ? k_scale : q_scale;
    const int half = rot >> 1;
    const int p = pos[t];
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float y;
        if (d < half) {
            const float c = cos_t[(size_t)p * half + d], s = sin_t[(size_t)p * half + d];
            y = to_f32(src[d]) * c - to_f32(src[d + half]) * s;
        } else if (d < rot) {
            const int i = d - half;
            const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
            y = to_f32(src[d]) * c + to_f32(src[i]) * s;
        } else {
            y = to_f32(src[d]);
        }
        dst[d] = y * scale;
    }
}

RB_EXPORT int rb_rotary_to_f32(const void* x, int ld, int q_off, int k_off, const float* cos_t, const float* sin_t,
                               int rot, const int* pos, float* q32, float* k32, int act_dtype, int T, int heads, int D,
                               float q_scale, float k_scale, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rot > D || (rot & 1)) return (int)cudaErrorInvalidValue;
    dim3 grid(T, 2 * heads);
    const int threads = D <= 32 ? 32 : D <= 64 ? 64 : 128;
    if (act_dtype == RB_F32)
        rb_launch_pdl(rotary_to_f32_kernel<float>, dim3(grid), dim3(threads), 0, st, (const float*)x, ld, q_off, k_off, cos_t, sin_t, rot, pos,
                                                             q32, k32, heads, D, q_scale, k_scale);
    else
        rb_launch_pdl(rotary_to_f32_kernel<bf16>, dim3(grid), dim3(threads), 0, st, (const bf16*)x, ld, q_off, k_off, cos_t, sin_t, rot, pos,
                                                            q32, k32, heads, D, q_scale, k_scale);
    return rb_launch_status();
}

// The same rotation in place, on the q and k heads of a packed [q heads | k heads | ...] row of the activation type,
// for rotary widths that the rotation-and-cache-write kernel does not take (any even width).  A thread owns a pair.
template <typename TA>
__global__ void rotary_inplace_kernel(TA* __restrict__ x, int ld, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int rot, const int* __restrict__ pos,
                                      int heads, int D) {
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;            // h over q heads, then k heads
    const int half = rot >> 1;
    TA* row = x + (size_t)t * ld + (size_t)h * D;
    const int p = pos[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
        const float u = to_f32(row[i]), v = to_f32(row[i + half]);
        row[i] = from_f32<TA>(u * c - v * s);
        row[i + half] = from_f32<TA>(v * c + u * s);
    }
}

RB_EXPORT int rb_rotary_inplace(void* x, int ld, const float* cos_t, const float* sin_t, int rot, const int* pos,
                                int act_dtype, int T, int heads, int D, cudaStream_t st) {
    if (T <= 0 || rot <= 0) return 0;
    if (rot > D || (rot & 1)) return (int)cudaErrorInvalidValue;
    dim3 grid(T, heads);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(rotary_inplace_kernel<float>, grid, dim3(32), 0, st, (float*)x, ld, cos_t, sin_t, rot, pos, heads, D);
    return rb_launch_pdl(rotary_inplace_kernel<bf16>, grid, dim3(32), 0, st, (bf16*)x, ld, cos_t, sin_t, rot, pos, heads, D);
}

// ---------------------------------------------------------------- what the delta rule needs of a token
// Units of work (blockIdx.y): G query heads, G key heads, H value heads, H rows of decays, one of betas.
//   q, k, v: a short causal convolution over time per channel (taps [C, K], the last column is the current
//   token's; what lies before the segment comes from the request's conv state, which holds the K - 1 inputs
//   before it, oldest first, and is zero for a new request), then silu; q and k heads are then made unit
//   vectors (x / sqrt(sum x^2 + 1e-6)), q also times q_scale.  Channels: q heads, k heads, v heads, in this order.
//   decay[t, h, i] = exp(-exp(A_log[h]) * softplus(a[t, h, i] + dt_bias[h, i]))   (in place over a; i < DA, which is D
//   for a decay per key row and 1 for one decay a head)
//   beta[t, h] = sigmoid(b[t, h])                                                 (in place over b)
template <typename TA>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const TA* __restrict__ x, int ld, const void* __restrict__ taps, int taps_dtype, int K,
                  const float* __restrict__ state, long long state_stride, int conv_off,
                  const int* __restrict__ tok_seg, const int* __restrict__ cu_q, const int* __restrict__ seg_slot,
                  float* __restrict__ q32, float* __restrict__ k32, float* __restrict__ v32,
                  float* __restrict__ a, const void* __restrict__ A_log, const void* __restrict__ dt_bias, int vec_dtype,
                  float* __restrict__ b, int H, int G, int D, int V, float q_scale, int DA) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x, unit = blockIdx.y;
    if (unit >= 2 * G + H) {
        if (unit < 2 * G + 2 * H) {
            const int h = unit - 2 * G - H;
            const float rate = expf(load_as_f32(A_log, vec_dtype, h));
            for (int i = threadIdx.x; i < DA; i += blockDim.x) {
                const size_t e = ((size_t)t * H + h) * DA + i;
                a[e] = expf(-rate * softplus_f(a[e] + load_as_f32(dt_bias, vec_dtype, (size_t)h * DA + i)));
            }
        } else {
            for (int h = threadIdx.x; h < H; h += blockDim.x) b[(size_t)t * H + h] = sigmoid_f(b[(size_t)t * H + h]);
        }
        return;
    }
    const int seg = tok_seg[t];
    const int l = t - cu_q[seg];                          // tokens of this segment before t
    const float* cs = state + (long long)seg_slot[seg] * state_stride + conv_off;
    int c0, len;
    float* dst;
    if (unit < G) { c0 = unit * D; len = D; dst = q32 + ((size_t)t * G + unit) * D; }
    else if (unit < 2 * G) { c0 = G * D + (unit - G) * D; len = D; dst = k32 + ((size_t)t * G + (unit - G)) * D; }
    else { c0 = 2 * G * D + (unit - 2 * G) * V; len = V; dst = v32 + ((size_t)t * H + (unit - 2 * G)) * V; }
    float ss = 0.f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const int c = c0 + i;
        float y = 0.f;
        for (int jb = K - 1; jb >= 0; --jb) {             // jb tokens back, oldest first
            const float w = load_as_f32(taps, taps_dtype, (size_t)c * K + (K - 1 - jb));
            const float xv = jb <= l ? to_f32(x[(size_t)(t - jb) * ld + c]) : cs[(size_t)c * (K - 1) + (K - 1 - (jb - l))];
            y = fmaf(w, xv, y);
        }
        y = y / (1.0f + expf(-y));
        dst[i] = y;
        ss += y * y;
    }
    if (unit < 2 * G) {
        ss = block_sum(ss, scratch);
        const float inv = (unit < G ? q_scale : 1.0f) / sqrtf(ss + 1e-6f);
        for (int i = threadIdx.x; i < len; i += blockDim.x) dst[i] *= inv;
    }
}

RB_EXPORT int rb_delta_prep(const void* x, int ld, const void* taps, int taps_dtype, int K, const float* state,
                            long long state_stride, int conv_off, const int* tok_seg, const int* cu_q, const int* seg_slot,
                            float* q32, float* k32, float* v32, float* a, const void* A_log, const void* dt_bias,
                            int vec_dtype, float* b, int act_dtype, int T, int H, int G, int D, int V, float q_scale,
                            int head_decay, cudaStream_t st) {
    if (T <= 0) return 0;
    if (K < 1) return (int)cudaErrorInvalidValue;
    const int DA = head_decay ? 1 : D;
    dim3 grid(T, 2 * G + 2 * H + 1);
    if (act_dtype == RB_F32)
        rb_launch_pdl(delta_prep_kernel<float>, dim3(grid), dim3(128), 0, st, (const float*)x, ld, taps, taps_dtype, K, state, state_stride, conv_off,
            tok_seg, cu_q, seg_slot, q32, k32, v32, a, A_log, dt_bias, vec_dtype, b, H, G, D, V, q_scale, DA);
    else
        rb_launch_pdl(delta_prep_kernel<bf16>, dim3(grid), dim3(128), 0, st, (const bf16*)x, ld, taps, taps_dtype, K, state, state_stride, conv_off,
            tok_seg, cu_q, seg_slot, q32, k32, v32, a, A_log, dt_bias, vec_dtype, b, H, G, D, V, q_scale, DA);
    return rb_launch_status();
}

// The conv state after a step: the last K - 1 inputs of each channel, oldest first.  A segment shorter than K - 1
// keeps the newest part of what the state held.  A thread reads all it needs of a channel before it writes.
#define CONV_MAX_TAPS 32
template <typename TA>
__global__ void conv_state_update_kernel(const TA* __restrict__ x, int ld, int K, float* __restrict__ state,
                                         long long state_stride, int conv_off, const int* __restrict__ cu_q,
                                         const int* __restrict__ seg_slot, int C) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int t0 = cu_q[seg], t1 = cu_q[seg + 1], L = t1 - t0;
    float* cs = state + (long long)seg_slot[seg] * state_stride + conv_off + (size_t)c * (K - 1);
    float keep[CONV_MAX_TAPS];
    for (int m = 0; m < K - 1; ++m) {
        const int back = K - 2 - m;                       // tokens before the segment's last one
        keep[m] = back < L ? to_f32(x[(size_t)(t1 - 1 - back) * ld + c]) : cs[K - 2 - (back - L)];
    }
    for (int m = 0; m < K - 1; ++m) cs[m] = keep[m];
}

RB_EXPORT int rb_conv_state_update(const void* x, int ld, int K, float* state, long long state_stride, int conv_off,
                                   const int* cu_q, const int* seg_slot, int act_dtype, int C, int segments,
                                   cudaStream_t st) {
    if (segments <= 0 || K <= 1) return 0;
    if (K - 1 > CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
    dim3 grid((C + 127) / 128, segments);
    if (act_dtype == RB_F32)
        rb_launch_pdl(conv_state_update_kernel<float>, dim3(grid), dim3(128), 0, st, (const float*)x, ld, K, state, state_stride, conv_off, cu_q, seg_slot, C);
    else
        rb_launch_pdl(conv_state_update_kernel<bf16>, dim3(grid), dim3(128), 0, st, (const bf16*)x, ld, K, state, state_stride, conv_off, cu_q, seg_slot, C);
    return rb_launch_status();
}

// ---------------------------------------------------------------- after the scan: per-head norm, weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * act(gate[t, h, :]), one warp a (token, head).
// w_mode 0: no weight; 1: a weight of size V shared by the heads; 2: a weight over all heads (H*V).
// gate_act 0: silu, 1: sigmoid.  The gate has the activation type and rows of stride gate_ld.
template <typename TA>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const TA* __restrict__ gate, int gate_ld,
                                      const void* __restrict__ w, int w_dtype, int w_mode, int gate_act, float eps,
                                      TA* __restrict__ out, int rows, int H, int V) {
    pdl_wait();
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int t = row / H, h = row - t * H;
    const float* x = o + (size_t)row * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)V + eps);
    const TA* g = gate + (size_t)t * gate_ld + (size_t)h * V;
    TA* y = out + (size_t)row * V;
    for (int i = lane; i < V; i += 32) {
        float val = x[i] * rstd;
        if (w_mode == 1) val *= load_as_f32(w, w_dtype, i);
        else if (w_mode == 2) val *= load_as_f32(w, w_dtype, (size_t)h * V + i);
        const float gv = to_f32(g[i]);
        val *= gate_act == 0 ? gv / (1.0f + expf(-gv)) : 1.0f / (1.0f + expf(-gv));
        y[i] = from_f32<TA>(val);
    }
}

RB_EXPORT int rb_head_norm_gate(const float* o, const void* gate, int gate_ld, const void* w, int w_dtype, int w_mode,
                                int gate_act, float eps, void* out, int act_dtype, int T, int H, int V, cudaStream_t st) {
    const int rows = T * H;
    if (rows <= 0) return 0;
    const int blocks = (rows + 3) / 4;
    if (act_dtype == RB_F32)
        rb_launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, st, o, (const float*)gate, gate_ld, w, w_dtype, w_mode, gate_act, eps,
                                                            (float*)out, rows, H, V);
    else
        rb_launch_pdl(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(128), 0, st, o, (const bf16*)gate, gate_ld, w, w_dtype, w_mode, gate_act, eps,
                                                           (bf16*)out, rows, H, V);
    return rb_launch_status();
}

// ---------------------------------------------------------------- residual add and one or two norms of the same row
// stream[t] += s1 * d1[t] + s2 * d2[t] (each delta may be absent; float32 or the activation type), then
// out1 = stream * rstd * (offset + w1) and, if asked for, out2 = stream * rstd * (offset + w2): the two norms of a
// block whose mixer and feed-forward read the same stream share the row's mean square.  Without out1 only the add
// is done.  With `rows` only the listed rows are normed and the stream is left as it is.
template <typename TA>
__global__ void __launch_bounds__(256)
add_dual_norm_kernel(float* __restrict__ stream, const void* __restrict__ d1, int d1_f32, float s1,
                     const void* __restrict__ d2, int d2_f32, float s2, const int* __restrict__ rows,
                     const void* __restrict__ w1, const void* __restrict__ w2, int w_dtype, float eps, float offset,
                     TA* __restrict__ out1, TA* __restrict__ out2, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = stream + t * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (d1 || d2) {
            float d = 0.f;
            if (d1) d = s1 * ld_elem(d1, d1_f32, t * H + i);
            if (d2) d = fmaf(s2, ld_elem(d2, d2_f32, t * H + i), d);
            v += d;
            if (!rows) xr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    if (!out1) return;
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (rows && (d1 || d2)) {                      // the stream was not written: add again
            float d = 0.f;
            if (d1) d = s1 * ld_elem(d1, d1_f32, t * H + i);
            if (d2) d = fmaf(s2, ld_elem(d2, d2_f32, t * H + i), d);
            v += d;
        }
        v *= rstd;
        out1[(size_t)r * H + i] = from_f32<TA>(v * (offset + load_as_f32(w1, w_dtype, i)));
        if (out2) out2[(size_t)r * H + i] = from_f32<TA>(v * (offset + load_as_f32(w2, w_dtype, i)));
    }
}

// The same with four columns a thread and round: 16-byte accesses of the stream and of float32 addends, 8-byte ones of
// bfloat16 addends and outputs.  Needs H % 4 == 0 and every pointer aligned to 16 bytes.
__device__ __forceinline__ float4 ld4_any(const void* p, int f32, size_t i) {      // four elements from element i (a multiple of 4)
    if (f32) return *reinterpret_cast<const float4*>((const float*)p + i);
    const uint2 raw = *reinterpret_cast<const uint2*>((const bf16*)p + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4_act(float* p, size_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void st4_act(bf16* p, size_t i, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a); raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p + i) = raw;
}

template <typename TA>
__global__ void __launch_bounds__(256)
add_dual_norm_vec_kernel(float* __restrict__ stream, const void* __restrict__ d1, int d1_f32, float s1,
                         const void* __restrict__ d2, int d2_f32, float s2, const int* __restrict__ rows,
                         const void* __restrict__ w1, const void* __restrict__ w2, int w_dtype, float eps, float offset,
                         TA* __restrict__ out1, TA* __restrict__ out2, int H) {
    __shared__ float scratch[33];
    pdl_wait();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = stream + t * H;
    auto summed = [&](int i) {                              // the row's columns i .. i + 3 with the addends
        float4 v = *reinterpret_cast<const float4*>(xr + i);
        if (d1) { const float4 d = ld4_any(d1, d1_f32, t * H + i); v.x = fmaf(s1, d.x, v.x); v.y = fmaf(s1, d.y, v.y); v.z = fmaf(s1, d.z, v.z); v.w = fmaf(s1, d.w, v.w); }
        if (d2) { const float4 d = ld4_any(d2, d2_f32, t * H + i); v.x = fmaf(s2, d.x, v.x); v.y = fmaf(s2, d.y, v.y); v.z = fmaf(s2, d.z, v.z); v.w = fmaf(s2, d.w, v.w); }
        return v;
    };
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        const float4 v = summed(i);
        if ((d1 || d2) && !rows) *reinterpret_cast<float4*>(xr + i) = v;
        ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    if (!out1) return;
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        // a thread reads back the columns it wrote itself; with `rows` the stream was not written: add again
        float4 v = rows ? summed(i) : *reinterpret_cast<const float4*>(xr + i);
        v.x *= rstd; v.y *= rstd; v.z *= rstd; v.w *= rstd;
        const float4 a = ld4_any(w1, w_dtype == RB_F32, i);
        st4_act(out1, (size_t)r * H + i, make_float4(v.x * (offset + a.x), v.y * (offset + a.y), v.z * (offset + a.z), v.w * (offset + a.w)));
        if (out2) {
            const float4 b = ld4_any(w2, w_dtype == RB_F32, i);
            st4_act(out2, (size_t)r * H + i, make_float4(v.x * (offset + b.x), v.y * (offset + b.y), v.z * (offset + b.z), v.w * (offset + b.w)));
        }
    }
}

RB_EXPORT int rb_add_dual_norm(float* stream, const void* d1, int d1_f32, float s1, const void* d2, int d2_f32, float s2,
                               const int* rows, const void* w1, const void* w2, int w_dtype, float eps, float offset,
                               void* out1, void* out2, int act_dtype, int n, int H, cudaStream_t st) {
    if (n <= 0) return 0;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (H % 4 == 0 && aligned(stream) && aligned(d1) && aligned(d2) && aligned(w1) && aligned(w2) && aligned(out1) && aligned(out2)) {
        if (act_dtype == RB_F32)
            return rb_launch_pdl(add_dual_norm_vec_kernel<float>, dim3(n), dim3(256), 0, st, stream, d1, d1_f32, s1, d2, d2_f32, s2, rows,
                                 w1, w2, w_dtype, eps, offset, (float*)out1, (float*)out2, H);
        return rb_launch_pdl(add_dual_norm_vec_kernel<bf16>, dim3(n), dim3(256), 0, st, stream, d1, d1_f32, s1, d2, d2_f32, s2, rows,
                             w1, w2, w_dtype, eps, offset, (bf16*)out1, (bf16*)out2, H);
    }
    if (act_dtype == RB_F32)
        rb_launch_pdl(add_dual_norm_kernel<float>, dim3(n), dim3(256), 0, st, stream, d1, d1_f32, s1, d2, d2_f32, s2, rows, w1, w2, w_dtype, eps,
                                                      offset, (float*)out1, (float*)out2, H);
    else
        rb_launch_pdl(add_dual_norm_kernel<bf16>, dim3(n), dim3(256), 0, st, stream, d1, d1_f32, s1, d2, d2_f32, s2, rows, w1, w2, w_dtype, eps,
                                                     offset, (bf16*)out1, (bf16*)out2, H);
    return rb_launch_status();
}

// ---------------------------------------------------------------- y = s1 * a + s2 * b, elementwise (sum of two mixers)
template <typename TO>
__global__ void scaled_sum_kernel(const void* __restrict__ a, int a_f32, float s1, const void* __restrict__ b, int b_f32,
                                  float s2, TO* __restrict__ y, size_t n) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = from_f32<TO>(fmaf(s2, ld_elem(b, b_f32, i), s1 * ld_elem(a, a_f32, i)));
}

RB_EXPORT int rb_scaled_sum(const void* a, int a_f32, float s1, const void* b, int b_f32, float s2, void* y, int out_f32,
                            long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (out_f32) rb_launch_pdl(scaled_sum_kernel<float>, dim3(blocks), dim3(256), 0, st, a, a_f32, s1, b, b_f32, s2, (float*)y, (size_t)n);
    else rb_launch_pdl(scaled_sum_kernel<bf16>, dim3(blocks), dim3(256), 0, st, a, a_f32, s1, b, b_f32, s2, (bf16*)y, (size_t)n);
    return rb_launch_status();
}

// ---------------------------------------------------------------- token shift: mixes of a token's input with its predecessor's
// out[n, t, :] = x[t] + (x[t-1] - x[t]) * mu[n], n < N, where x[t-1] of a segment's first token is the request's kept
// row (state + shift_off: the last input of the step before, zero for a new request).  Float32 arithmetic.
template <typename TA>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(const TA* __restrict__ x, int ld, const void* __restrict__ mu, int mu_dtype, int N,
                       const float* __restrict__ state, long long state_stride, int shift_off,
                       const int* __restrict__ tok_seg, const int* __restrict__ cu_q, const int* __restrict__ seg_slot,
                       TA* __restrict__ out, int T, int W) {
    pdl_wait();
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    const bool first = t == cu_q[seg];
    const float* kept = state + (long long)seg_slot[seg] * state_stride + shift_off;
    const TA* cur = x + (size_t)t * ld;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {   // a column a thread
        const float c = to_f32(cur[i]);
        const float d = (first ? kept[i] : to_f32(x[(size_t)(t - 1) * ld + i])) - c;
        for (int n = 0; n < N; ++n)
            out[((size_t)n * T + t) * W + i] = from_f32<TA>(fmaf(d, load_as_f32(mu, mu_dtype, (size_t)n * W + i), c));
    }
}

RB_EXPORT int rb_token_shift_mix(const void* x, int ld, const void* mu, int mu_dtype, int N, const float* state,
                                 long long state_stride, int shift_off, const int* tok_seg, const int* cu_q,
                                 const int* seg_slot, void* out, int act_dtype, int T, int W, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    const int threads = 128;
    const int across = (W + threads - 1) / threads < 65535 ? (W + threads - 1) / threads : 65535;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(token_shift_mix_kernel<float>, dim3(T, across), dim3(threads), 0, st, (const float*)x, ld, mu, mu_dtype, N,
                             state, state_stride, shift_off, tok_seg, cu_q, seg_slot, (float*)out, T, W);
    return rb_launch_pdl(token_shift_mix_kernel<bf16>, dim3(T, across), dim3(threads), 0, st, (const bf16*)x, ld, mu, mu_dtype, N, state,
                         state_stride, shift_off, tok_seg, cu_q, seg_slot, (bf16*)out, T, W);
}

// ---------------------------------------------------------------- what the state-space scan needs of a token
// x: rows of a projection buffer; C channels from column c_off pass a short causal convolution over time (taps [C, K],
// the last column is the current token's; what lies before the segment comes from the request's conv state, which
// holds the K - 1 inputs before it, oldest first, and is zero for a new request), plus a bias per channel, then silu;
// the results go to conv_out [T, C] in float32.  H step sizes from column dt_off:
//     dt[t, h] = softplus(x[t, dt_off + h] + dt_bias[h]),   decay[t, h] = exp(-exp(A_log[h]) * dt[t, h]).
// blockIdx.y < gridDim.y - 1: a run of 256 channels; the last: the steps and decays.
template <typename TA>
__global__ void __launch_bounds__(256)
ssm_prep_kernel(const TA* __restrict__ x, int ld, int c_off, int C, const void* __restrict__ taps, const void* __restrict__ bias,
                int taps_dtype, int K, const float* __restrict__ state, long long state_stride, int conv_off,
                const int* __restrict__ tok_seg, const int* __restrict__ cu_q, const int* __restrict__ seg_slot,
                float* __restrict__ conv_out, int dt_off, int H, const void* __restrict__ dt_bias,
                const void* __restrict__ A_log, int vec_dtype, float* __restrict__ dt, float* __restrict__ decay) {
    pdl_wait();
    const int t = blockIdx.x;
    if (blockIdx.y == gridDim.y - 1) {
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float step = softplus_f(to_f32(x[(size_t)t * ld + dt_off + h]) + load_as_f32(dt_bias, vec_dtype, h));
            dt[(size_t)t * H + h] = step;
            decay[(size_t)t * H + h] = expf(-expf(load_as_f32(A_log, vec_dtype, h)) * step);
        }
        return;
    }
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seg = tok_seg[t];
    const int l = t - cu_q[seg];                          // tokens of this segment before t
    const float* cs = state + (long long)seg_slot[seg] * state_stride + conv_off + (size_t)c * (K - 1);
    float y = 0.f;
    for (int jb = K - 1; jb >= 0; --jb) {                 // jb tokens back, oldest first
        const float w = load_as_f32(taps, taps_dtype, (size_t)c * K + (K - 1 - jb));
        const float xv = jb <= l ? to_f32(x[(size_t)(t - jb) * ld + c_off + c]) : cs[K - 1 - (jb - l)];
        y = fmaf(w, xv, y);
    }
    y += load_as_f32(bias, taps_dtype, c);
    conv_out[(size_t)t * C + c] = y / (1.0f + expf(-y));
}

RB_EXPORT int rb_ssm_prep(const void* x, int ld, int c_off, int C, const void* taps, const void* bias, int taps_dtype, int K,
                          const float* state, long long state_stride, int conv_off, const int* tok_seg, const int* cu_q,
                          const int* seg_slot, float* conv_out, int dt_off, int H, const void* dt_bias, const void* A_log,
                          int vec_dtype, float* dt, float* decay, int act_dtype, int T, cudaStream_t st) {
    if (T <= 0) return 0;
    if (K < 1 || C <= 0) return (int)cudaErrorInvalidValue;
    dim3 grid(T, (C + 255) / 256 + 1);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(ssm_prep_kernel<float>, grid, dim3(256), 0, st, (const float*)x, ld, c_off, C, taps, bias, taps_dtype, K,
                             state, state_stride, conv_off, tok_seg, cu_q, seg_slot, conv_out, dt_off, H, dt_bias, A_log,
                             vec_dtype, dt, decay);
    return rb_launch_pdl(ssm_prep_kernel<bf16>, grid, dim3(256), 0, st, (const bf16*)x, ld, c_off, C, taps, bias, taps_dtype, K, state,
                         state_stride, conv_off, tok_seg, cu_q, seg_slot, conv_out, dt_off, H, dt_bias, A_log, vec_dtype, dt,
                         decay);
}

// ---------------------------------------------------------------- after the scan: gate first, then a norm over equal parts
// v = y * silu(z); out[t, p, :] = v / sqrt(mean over the part (v^2) + eps) * w: a row of `width` values is normed in
// `parts` equal parts, each by its own root mean square.  One warp a (token, part); the gate has the activation type
// and rows of stride z_ld.
template <typename TA>
__global__ void gated_part_norm_kernel(const float* __restrict__ y, const TA* __restrict__ z, int z_ld,
                                       const void* __restrict__ w, int w_dtype, float eps, TA* __restrict__ out, int rows,
                                       int parts, int size) {
    pdl_wait();
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int t = row / parts, p = row - t * parts;
    const float* yr = y + (size_t)row * size;
    const TA* zr = z + (size_t)t * z_ld + (size_t)p * size;
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) {
        const float g = to_f32(zr[i]);
        const float v = yr[i] * (g / (1.0f + expf(-g)));
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)size + eps);
    TA* o = out + (size_t)row * size;
    for (int i = lane; i < size; i += 32) {
        const float g = to_f32(zr[i]);
        const float v = yr[i] * (g / (1.0f + expf(-g)));
        o[i] = from_f32<TA>(v * rstd * load_as_f32(w, w_dtype, (size_t)p * size + i));
    }
}

// The same for parts of 256 elements or more: one CTA of 128 threads a part, the first eight gated values of a thread
// kept in registers between the sum of squares and the store.  Which of the two kernels runs depends on the part's size
// alone, never on the number of rows, so a row's sums are added in one order whatever else the step holds.
#define PART_NORM_WIDE_FROM 256
template <typename TA>
__global__ void __launch_bounds__(128)
gated_part_norm_wide_kernel(const float* __restrict__ y, const TA* __restrict__ z, int z_ld,
                            const void* __restrict__ w, int w_dtype, float eps, TA* __restrict__ out, int parts, int size) {
    __shared__ float scratch[33];
    constexpr int HOLD = 8;
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const int t = row / parts, p = row - t * parts;
    const float* yr = y + (size_t)row * size;
    const TA* zr = z + (size_t)t * z_ld + (size_t)p * size;
    float held[HOLD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < HOLD; ++j) {
        const int i = tid + j * 128;
        held[j] = 0.f;
        if (i < size) {
            const float g = to_f32(zr[i]);
            held[j] = yr[i] * (g / (1.0f + expf(-g)));
            ss = fmaf(held[j], held[j], ss);
        }
    }
    for (int i = tid + HOLD * 128; i < size; i += 128) {
        const float g = to_f32(zr[i]);
        const float v = yr[i] * (g / (1.0f + expf(-g)));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    pdl_trigger_late();
    const float rstd = 1.0f / sqrtf(ss / (float)size + eps);
    TA* o = out + (size_t)row * size;
#pragma unroll
    for (int j = 0; j < HOLD; ++j) {
        const int i = tid + j * 128;
        if (i < size) o[i] = from_f32<TA>(held[j] * rstd * load_as_f32(w, w_dtype, (size_t)p * size + i));
    }
    for (int i = tid + HOLD * 128; i < size; i += 128) {
        const float g = to_f32(zr[i]);
        const float v = yr[i] * (g / (1.0f + expf(-g)));
        o[i] = from_f32<TA>(v * rstd * load_as_f32(w, w_dtype, (size_t)p * size + i));
    }
}

RB_EXPORT int rb_gated_part_norm(const float* y, const void* z, int z_ld, const void* w, int w_dtype, float eps, void* out,
                                 int act_dtype, int T, int parts, int size, cudaStream_t st) {
    const int rows = T * parts;
    if (rows <= 0) return 0;
    if (size >= PART_NORM_WIDE_FROM) {
        if (act_dtype == RB_F32)
            return rb_launch_pdl(gated_part_norm_wide_kernel<float>, dim3(rows), dim3(128), 0, st, y, (const float*)z, z_ld, w,
                                 w_dtype, eps, (float*)out, parts, size);
        return rb_launch_pdl(gated_part_norm_wide_kernel<bf16>, dim3(rows), dim3(128), 0, st, y, (const bf16*)z, z_ld, w, w_dtype,
                             eps, (bf16*)out, parts, size);
    }
    const int blocks = (rows + 3) / 4;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(gated_part_norm_kernel<float>, dim3(blocks), dim3(128), 0, st, y, (const float*)z, z_ld, w, w_dtype, eps,
                             (float*)out, rows, parts, size);
    return rb_launch_pdl(gated_part_norm_kernel<bf16>, dim3(blocks), dim3(128), 0, st, y, (const bf16*)z, z_ld, w, w_dtype, eps,
                         (bf16*)out, rows, parts, size);
}

// ---------------------------------------------------------------- gated linear recurrence per channel
// A recurrent branch of `W` channels beside a gate branch:  u = conv(x + x_bias) + conv_bias (a causal convolution
// over time per channel, taps [W, K] with the last column for the token itself; what lies before position 0 is zero,
// what lies before the step comes from the request's held inputs, which are kept without the bias);  with gate
// pre-activations r~, i~ (block-diagonal maps of u, computed outside; float32 [2][blocks][T][block size]):  r = sigmoid(r~ + rb), i = sigmoid(i~ + ib),
// log f = -c r softplus(lam), s <- f s + sqrt(1 - f^2) i u, out = s * gelu_tanh(y + y_bias).  Everything from the
// gates on is float32; the state s [W] of a request lives in its slot and starts at zero.
template <typename TA>
__global__ void __launch_bounds__(128)
gated_conv_kernel(const TA* __restrict__ x, int ld, const void* __restrict__ x_bias, const void* __restrict__ taps,
                  const void* __restrict__ conv_bias, int w_dtype, int K, const float* __restrict__ state,
                  long long state_stride, int conv_off, const int* __restrict__ pos, const int* __restrict__ tok_seg,
                  const int* __restrict__ cu_q, const int* __restrict__ seg_slot, TA* __restrict__ u, int W) {
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int seg = tok_seg[t];
    const int l = t - cu_q[seg], p = pos[t];
    const float* cs = state + (long long)seg_slot[seg] * state_stride + conv_off + (size_t)c * (K - 1);
    const float xb = x_bias ? load_as_f32(x_bias, w_dtype, c) : 0.f;
    float y = conv_bias ? load_as_f32(conv_bias, w_dtype, c) : 0.f;
    for (int jb = K - 1; jb >= 0; --jb) {                  // jb tokens back, oldest first
        if (jb > p) continue;                              // before the sequence: nothing
        const float w = load_as_f32(taps, w_dtype, (size_t)c * K + (K - 1 - jb));
        const float xv = jb <= l ? to_f32(x[(size_t)(t - jb) * ld + c]) : cs[K - 1 - (jb - l)];
        y = fmaf(w, xv + xb, y);
    }
    u[(size_t)t * W + c] = from_f32<TA>(y);
}

RB_EXPORT int rb_gated_conv(const void* x, int ld, const void* x_bias, const void* taps, const void* conv_bias, int w_dtype,
                            int K, const float* state, long long state_stride, int conv_off, const int* pos,
                            const int* tok_seg, const int* cu_q, const int* seg_slot, void* u, int act_dtype, int T, int W,
                            cudaStream_t st) {
    if (T <= 0) return 0;
    if (K < 1) return (int)cudaErrorInvalidValue;
    dim3 grid(T, (W + 127) / 128);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(gated_conv_kernel<float>, grid, dim3(128), 0, st, (const float*)x, ld, x_bias, taps, conv_bias, w_dtype, K,
                             state, state_stride, conv_off, pos, tok_seg, cu_q, seg_slot, (float*)u, W);
    return rb_launch_pdl(gated_conv_kernel<bf16>, grid, dim3(128), 0, st, (const bf16*)x, ld, x_bias, taps, conv_bias, w_dtype, K,
                         state, state_stride, conv_off, pos, tok_seg, cu_q, seg_slot, (bf16*)u, W);
}

// One thread a channel walks its segment's tokens in order; the loads of RU tokens are issued before the first is used.
#define GLR_UNROLL 8
template <typename TA>
__global__ void __launch_bounds__(128)
gated_recurrence_kernel(const TA* __restrict__ u, const float* __restrict__ gates, int bs, const void* __restrict__ r_bias,
                        const void* __restrict__ i_bias, const void* __restrict__ lam, int w_dtype, float c_decay,
                        const TA* __restrict__ y, int y_ld, const void* __restrict__ y_bias, float* __restrict__ state,
                        long long state_stride, int s_off, const int* __restrict__ cu_q, const int* __restrict__ seg_slot,
                        TA* __restrict__ out, int W, int T, float* __restrict__ log_decay) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int t0 = cu_q[seg], t1 = cu_q[seg + 1];
    float* sp = state + (long long)seg_slot[seg] * state_stride + s_off + c;
    float s = *sp;
    const int blk = c / bs, o = c - blk * bs;
    const float* g_r = gates + (size_t)blk * T * bs + o;
    const float* g_i = g_r + (size_t)W * T;
    const float rb = load_as_f32(r_bias, w_dtype, c), ib = load_as_f32(i_bias, w_dtype, c);
    const float sp_lam = softplus_f(load_as_f32(lam, w_dtype, c));
    const float yb = y_bias ? load_as_f32(y_bias, w_dtype, c) : 0.f;
    float lf_sum = 0.f;
    for (int tc = t0; tc < t1; tc += GLR_UNROLL) {
        float ru[GLR_UNROLL], rr[GLR_UNROLL], ri[GLR_UNROLL], ry[GLR_UNROLL];
#pragma unroll
        for (int k = 0; k < GLR_UNROLL; ++k) {
            const size_t t = (size_t)min(tc + k, t1 - 1);
            ru[k] = to_f32(u[t * W + c]);
            rr[k] = g_r[t * bs];
            ri[k] = g_i[t * bs];
            ry[k] = to_f32(y[t * y_ld + c]);
        }
#pragma unroll
        for (int k = 0; k < GLR_UNROLL; ++k) {
            if (tc + k < t1) {
                const float r = sigmoid_f(rr[k] + rb), ig = sigmoid_f(ri[k] + ib);
                const float lf = -c_decay * r * sp_lam;
                const float f = expf(lf);
                lf_sum += lf;
                s = fmaf(f, s, sqrtf(-expm1f(2.f * lf)) * ig * ru[k]);
                out[(size_t)(tc + k) * W + c] = from_f32<TA>(s * rb_activate(ACT_GELU_TANH, ry[k] + yb, nullptr, 0, 0));
            }
        }
    }
    *sp = s;
    if (log_decay) log_decay[(size_t)seg * W + c] = lf_sum;     // the segment's transition is exp of this
}

// A long segment cut into pieces that were walked side by side from zero: per segment and channel, in order,
// pieces[p] <- carry; carry <- exp(log_decay[p]) * carry + pieces[p], starting from the request's state and leaving the
// last carry there.  A second walk of the pieces from those states gives the outputs.
__global__ void __launch_bounds__(128)
gated_pieces_combine_kernel(float* __restrict__ pieces, const float* __restrict__ log_decay, float* __restrict__ state,
                            long long state_stride, int s_off, const int* __restrict__ seg_first,
                            const int* __restrict__ seg_slot, int W) {
    pdl_wait();
    const int seg = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    float* sp = state + (long long)seg_slot[seg] * state_stride + s_off + c;
    float carry = *sp;
    for (int p = seg_first[seg]; p < seg_first[seg + 1]; ++p) {
        const size_t e = (size_t)p * W + c;
        const float own = pieces[e];
        pieces[e] = carry;
        carry = fmaf(expf(log_decay[e]), carry, own);
    }
    *sp = carry;
}

RB_EXPORT int rb_gated_pieces_combine(float* pieces, const float* log_decay, float* state, long long state_stride, int s_off,
                                      const int* seg_first, const int* seg_slot, int W, int segments, cudaStream_t st) {
    if (segments <= 0) return 0;
    return rb_launch_pdl(gated_pieces_combine_kernel, dim3((W + 127) / 128, segments), dim3(128), 0, st, pieces, log_decay, state,
                         state_stride, s_off, seg_first, seg_slot, W);
}

RB_EXPORT int rb_gated_recurrence(const void* u, const float* gates, int bs, const void* r_bias, const void* i_bias,
                                  const void* lam, int w_dtype, float c_decay, const void* y, int y_ld, const void* y_bias,
                                  float* state, long long state_stride, int s_off, const int* cu_q, const int* seg_slot,
                                  void* out, int act_dtype, int W, int T, int segments, float* log_decay, cudaStream_t st) {
    if (segments <= 0) return 0;
    if (bs <= 0 || W % bs) return (int)cudaErrorInvalidValue;
    dim3 grid((W + 127) / 128, segments);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(gated_recurrence_kernel<float>, grid, dim3(128), 0, st, (const float*)u, gates, bs, r_bias, i_bias, lam,
                             w_dtype, c_decay, (const float*)y, y_ld, y_bias, state, state_stride, s_off, cu_q, seg_slot,
                             (float*)out, W, T, log_decay);
    return rb_launch_pdl(gated_recurrence_kernel<bf16>, grid, dim3(128), 0, st, (const bf16*)u, gates, bs, r_bias, i_bias, lam,
                         w_dtype, c_decay, (const bf16*)y, y_ld, y_bias, state, state_stride, s_off, cu_q, seg_slot, (bf16*)out, W, T, log_decay);
}
