// Attention over cached latent rows: the kernels that are particular to it.
//
// A token leaves one row in the cache: [c (C numbers) | r (R numbers)], c a normed latent from which every
// head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c) and r a rotated key part that all
// heads share.  A head's score of query (a | b) against a token is  a . (Uk_h c) + b . r  =  (Uk_h^T a) . c + b . r,
// so with the query mapped once to q' = (Uk_h^T a | b) every head reads the same rows (keys of C + R numbers,
// values their first C numbers) and its output Uv_h (sum_j p_j c_j) is mapped back afterwards.
//
//   tb_latent_rows     from the 32-bit partial sums of the down projection: c = rms-normed first C columns
//                      times a weight, r = the last R columns rotated at the token's position (rotate-half
//                      pairing over the first rot_dims of them), times rot_scale; the row goes to the paged cache
//                      (a ring of ring_rows rows per sequence if that is set) and to a
//                      packed matrix; all arithmetic 32-bit, the row rounded once
//   tb_head_linear     y[t, h, :] = W[h] x[t, h, :] for per-head matrices W [heads][out][in]
//   tb_latent_decode   one query per sequence and head against the cached rows, the key range cut into
//                      splits; softmax with a sink: the denominator also holds exp(sink_h), which has no
//                      key and no value; partial (max, sum, o) per split are folded in split order
#include "common.cuh"

TB_EXPORT_ERROR()

struct LatentRowsArgs {
    const float* dkv; int splits; long long split_stride;     // [splits][T][C + R]
    const float* norm_w; float eps;                            // [C]
    const float* inv_freq; int rot_dims;                       // [rot_dims / 2]
    int C, R, n_tokens;
    const int* positions; const int* token_seq;
    const int* page_table; int pt_stride; int page_rows;
    void* pool;                                                // [pages][page_rows][C + R]
    void* rows;                                                // [T][C + R]
    int ring_rows; const int* len_after;                       // ring_rows > 0: row = position mod ring_rows, and only the
                                                               // last ring_rows tokens of a sequence ([batch] lengths) are cached
    float rot_scale;                                           // the rotated part comes times this
    long long row_stride;                                      // numbers between two tokens' rows of dkv (0: C + R)
    // the same product may carry, behind the C + R columns, a latent of the queries (Q columns, RMS-normed times
    // q_norm_w with the same eps, written to cq_out [T][Q] in the output's dtype) and n_gate gate columns (their
    // sigmoid goes to gate_out [T][n_gate], 32-bit)
    int Q; const float* q_norm_w; void* cq_out;
    int n_gate; float* gate_out;
};

template <typename T>
__global__ void __launch_bounds__(1024) latent_rows_kernel(LatentRowsArgs a) {
    pdl_launch_dependents();
    extern __shared__ float row_s[];
    __shared__ float red[33];
    const int t = blockIdx.x, W = a.C + a.R, WA = W + a.Q + a.n_gate;
    const size_t rs = a.row_stride > 0 ? (size_t)a.row_stride : (size_t)W;
    pdl_wait();
    float sq = 0.f, sq_q = 0.f;
    for (int c = threadIdx.x; c < WA; c += blockDim.x) {
        const float* src = a.dkv + (size_t)t * rs + c;
        float v = 0.f;
        int s = 0;
        for (; s + 4 <= a.splits; s += 4) {            // four loads on their way at a time, added in split order
            const float v0 = src[(size_t)s * a.split_stride], v1 = src[(size_t)(s + 1) * a.split_stride];
            const float v2 = src[(size_t)(s + 2) * a.split_stride], v3 = src[(size_t)(s + 3) * a.split_stride];
            v = (((v + v0) + v1) + v2) + v3;
        }
        for (; s < a.splits; s++) v += src[(size_t)s * a.split_stride];
        row_s[c] = v;
        if (c < a.C) sq = fmaf(v, v, sq);
        else if (c >= W && c < W + a.Q) sq_q = fmaf(v, v, sq_q);
    }
    const float rinv = 1.f / sqrtf(block_sum(sq, red) / (float)a.C + a.eps);     // its barriers also publish row_s
    if (a.Q > 0) {
        const float qinv = 1.f / sqrtf(block_sum(sq_q, red) / (float)a.Q + a.eps);
        T* cq = (T*)a.cq_out + (size_t)t * a.Q;
        for (int c = threadIdx.x; c < a.Q; c += blockDim.x) cq[c] = from_f<T>(row_s[W + c] * qinv * a.q_norm_w[c]);
    }
    for (int c = threadIdx.x; c < a.n_gate; c += blockDim.x)
        a.gate_out[(size_t)t * a.n_gate + c] = 1.f / (1.f + expf(-row_s[W + a.Q + c]));
    const int pos = a.positions[t];
    const int b = a.token_seq[t];
    const int crow = a.ring_rows > 0 ? pos % a.ring_rows : pos;
    const bool keep = a.ring_rows <= 0 || pos >= a.len_after[b] - a.ring_rows;
    const int page = keep ? a.page_table[(size_t)b * a.pt_stride + crow / a.page_rows] : 0;
    T* cache = (T*)a.pool + ((size_t)page * a.page_rows + crow % a.page_rows) * W;
    T* out = (T*)a.rows + (size_t)t * W;
    const int half = a.rot_dims / 2;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v;
        if (c < a.C) {
            v = row_s[c] * rinv * a.norm_w[c];
        } else {
            const int i = c - a.C;
            if (i < half) {
                float sn, cs; sincosf((float)pos * a.inv_freq[i], &sn, &cs);
                v = (row_s[c] * cs - row_s[c + half] * sn) * a.rot_scale;
            } else if (i < 2 * half) {
                float sn, cs; sincosf((float)pos * a.inv_freq[i - half], &sn, &cs);
                v = (row_s[c] * cs + row_s[c - half] * sn) * a.rot_scale;
            } else {
                v = row_s[c];
            }
        }
        const T r = from_f<T>(v);
        if (keep) cache[c] = r;
        out[c] = r;
    }
}

// ---------------------------------------------------------------------------
constexpr int HL_TOK = 8, HL_ROWS = 4;

// y[t, h, o] = sum_i w[h, o, i] x[t, h, i]: eight tokens per CTA (their x in shared memory), a warp per group of four
// output rows whose weights are on their way together, 16 bytes per lane and load where the row allows it.
template <typename T>
__global__ void __launch_bounds__(128) head_linear_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w,
                                                          T* __restrict__ y, long long y_stride, int n_tokens, int in, int out) {
    pdl_launch_dependents();
    extern __shared__ float x_s[];                      // [HL_TOK][in]
    const int h = blockIdx.y, t0 = blockIdx.x * HL_TOK;
    const int nt = min(HL_TOK, n_tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < HL_TOK * in; i += blockDim.x) {
        const int tt = i / in, c = i % in;
        x_s[i] = tt < nt ? to_f<T>(x[(size_t)(t0 + tt) * x_stride + (size_t)h * in + c]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * out * in;
    constexpr int VEC = 16 / sizeof(T);
    const bool vec = (in % VEC) == 0 && (((uintptr_t)wh) & 15) == 0;
    for (int o0 = (blockIdx.z * nwarp + warp) * HL_ROWS; o0 < out; o0 += gridDim.z * nwarp * HL_ROWS) {
        float acc[HL_ROWS][HL_TOK];
#pragma unroll
        for (int r = 0; r < HL_ROWS; r++)
#pragma unroll
            for (int tt = 0; tt < HL_TOK; tt++) acc[r][tt] = 0.f;
        if (vec) {
            for (int c = lane * VEC; c < in; c += 32 * VEC) {
                uint4 wv[HL_ROWS];
#pragma unroll
                for (int r = 0; r < HL_ROWS; r++)
                    wv[r] = (o0 + r < out) ? *(const uint4*)(wh + (size_t)(o0 + r) * in + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int r = 0; r < HL_ROWS; r++) {
                    const T* e = (const T*)&wv[r];
#pragma unroll
                    for (int k = 0; k < VEC; k++) {
                        const float wf = to_f<T>(e[k]);
#pragma unroll
                        for (int tt = 0; tt < HL_TOK; tt++) acc[r][tt] = fmaf(wf, x_s[tt * in + c + k], acc[r][tt]);
                    }
                }
            }
        } else {
            for (int c = lane; c < in; c += 32) {
#pragma unroll
                for (int r = 0; r < HL_ROWS; r++) {
                    const float wf = (o0 + r < out) ? to_f<T>(wh[(size_t)(o0 + r) * in + c]) : 0.f;
#pragma unroll
                    for (int tt = 0; tt < HL_TOK; tt++) acc[r][tt] = fmaf(wf, x_s[tt * in + c], acc[r][tt]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < HL_ROWS; r++)
#pragma unroll
            for (int tt = 0; tt < HL_TOK; tt++) {
                const float sum = warp_sum(acc[r][tt]);
                if (lane == 0 && tt < nt && o0 + r < out) y[(size_t)(t0 + tt) * y_stride + (size_t)h * out + o0 + r] = from_f<T>(sum);
            }
    }
}

extern "C" int tb_head_linear(const void* x, long long x_stride, const void* w, void* y, long long y_stride, int dtype,
                              int n_tokens, int heads, int in, int out, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || in <= 0 || out <= 0 || in > 1536)
        return tb_refuse("head_linear: heads=%d in=%d out=%d (in at most 1536)", heads, in, out);
    int zs = (out + 4 * HL_ROWS - 1) / (4 * HL_ROWS);          // a CTA's four warps take 16 rows a round
    if (zs > 64) zs = 64;
    dim3 grid((n_tokens + HL_TOK - 1) / HL_TOK, heads, zs);
    TB_DISPATCH_1(dtype, T, tb_launch(head_linear_kernel<T>, dim3(grid), dim3(128), (size_t)HL_TOK * in * sizeof(float), stream,
                                      (const T*)x, x_stride, (const T*)w, (T*)y, y_stride, n_tokens, in, out));
    return tb_launch_status();
}

extern "C" int tb_latent_rows(const LatentRowsArgs* args, int dtype, cudaStream_t stream) {
    const LatentRowsArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.C <= 0 || a.R < 0 || a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.R || a.page_rows <= 0)
        return tb_refuse("latent_rows: C=%d R=%d rot_dims=%d page_rows=%d", a.C, a.R, a.rot_dims, a.page_rows);
    if (a.Q < 0 || a.n_gate < 0 || (a.Q > 0 && (a.q_norm_w == nullptr || a.cq_out == nullptr)) || (a.n_gate > 0 && a.gate_out == nullptr))
        return tb_refuse("latent_rows: Q=%d gate=%d need their outputs", a.Q, a.n_gate);
    if (a.ring_rows > 0 && (a.ring_rows % a.page_rows || a.len_after == nullptr))
        return tb_refuse("latent_rows: a ring of %d rows needs whole pages and the sequences' lengths", a.ring_rows);
    // few tokens (a decode step) are a chain of memory waits per thread: eight times the threads a token shorten it
    const int threads = a.n_tokens <= 2 * 148 ? 1024 : 128;
    TB_DISPATCH_1(dtype, T, tb_launch(latent_rows_kernel<T>, dim3(a.n_tokens), dim3(threads),
                                      (size_t)(a.C + a.R + a.Q + a.n_gate) * sizeof(float), stream, a));
    return tb_launch_status();
}

// ---------------------------------------------------------------------------
struct LatentDecodeArgs {
    const void* q; long long q_stride;                 // [batch] rows of heads * (C + R): the mapped queries
    const void* pool;                                  // [pages][page_rows][C + R]
    const int* page_table; int pt_stride; int page_rows;
    const int* len_after;                              // [batch] rows in the cache, the new token's included
    const float* sink;                                 // [heads] or null
    void* out; long long out_stride;                   // [batch] rows of heads * out_dim; the first C of a head are written
    float* partial;                                    // [batch][heads][splits][C + 2] when splits > 1
    int heads, C, R, out_dim, n_splits;
    float scale;
    int window;                                        // 0: every earlier row; W: the last W rows, the query's own included
    int ring_rows;                                     // 0: row = position; else row = position mod ring_rows
};

__device__ __forceinline__ int latent_first_key(int window, int len) { return (window > 0 && len > window) ? len - window : 0; }

template <int NC>
struct LatAcc {
    float m, l, o[NC];
    __device__ void init() { m = -INFINITY; l = 0.f;
#pragma unroll
        for (int c = 0; c < NC; c++) o[c] = 0.f; }
};

template <typename T, int NC>
__global__ void __launch_bounds__(128) latent_decode_kernel(LatentDecodeArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int KD = a.C + a.R, C = a.C;
    float* q_s = smem;                                 // [KD]
    float* red = smem + KD;                            // [nwarp][C + 2]
    pdl_wait();
    const T* qrow = (const T*)a.q + (size_t)b * a.q_stride + (size_t)h * KD;
    for (int e = threadIdx.x; e < KD; e += blockDim.x) q_s[e] = to_f<T>(qrow[e]);
    __syncthreads();
    const int len = a.len_after[b];
    const int lo = latent_first_key(a.window, len), lo32 = lo & ~31;
    int per = (len - lo32 + a.n_splits - 1) / a.n_splits;
    per = (per + 31) & ~31;
    const int beg = lo32 + split * per, end = min(len, beg + per);
    const int* pt = a.page_table + (size_t)b * a.pt_stride;

    LatAcc<NC> acc; acc.init();
    for (int j0 = beg + warp * 32; j0 < end; j0 += nwarp * 32) {
        const int j = j0 + lane;
        const bool valid = j < end && j >= lo;
        const T* krow = nullptr;
        float s = -INFINITY;
        if (valid) {
            const int r = a.ring_rows > 0 ? j % a.ring_rows : j;
            krow = (const T*)a.pool + ((size_t)pt[r / a.page_rows] * a.page_rows + (r % a.page_rows)) * KD;
            float d = 0.f;
            for (int e = 0; e < KD; e++) d = fmaf(q_s[e], to_f<T>(krow[e]), d);
            s = d * a.scale;
        }
        const float cm = warp_max(s);
        if (cm == -INFINITY) continue;                 // 32 rows before the window's first
        const float m_new = fmaxf(acc.m, cm);
        const float corr = (acc.m == -INFINITY) ? 0.f : expf(acc.m - m_new);
        const float p = valid ? expf(s - m_new) : 0.f;
        acc.l = acc.l * corr + warp_sum(p);
        acc.m = m_new;
#pragma unroll
        for (int c = 0; c < NC; c++) acc.o[c] *= corr;
        for (int jj = 0; jj < 32; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)krow, jj);
            if (pj == 0.f) continue;
            const T* v = (const T*)(uintptr_t)vp;
#pragma unroll
            for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < C) acc.o[c] = fmaf(pj, to_f<T>(v[d]), acc.o[c]); }
        }
    }
    float* mine = red + (size_t)warp * (C + 2);
    if (lane == 0) { mine[C] = acc.m; mine[C + 1] = acc.l; }
#pragma unroll
    for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < C) mine[d] = acc.o[c]; }
    __syncthreads();
    const float sink = (a.sink != nullptr) ? a.sink[h] : -INFINITY;
    float M = (a.n_splits == 1) ? sink : -INFINITY;
    for (int w = 0; w < nwarp; w++) M = fmaxf(M, red[(size_t)w * (C + 2) + C]);
    float L = 0.f;
    for (int w = 0; w < nwarp; w++) {
        const float mw = red[(size_t)w * (C + 2) + C];
        if (mw != -INFINITY) L += red[(size_t)w * (C + 2) + C + 1] * expf(mw - M);
    }
    if (a.n_splits == 1 && sink != -INFINITY) L += expf(sink - M);
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < nwarp; w++) {
            const float mw = red[(size_t)w * (C + 2) + C];
            if (mw != -INFINITY) o += red[(size_t)w * (C + 2) + d] * expf(mw - M);
        }
        if (a.n_splits == 1) ((T*)a.out)[(size_t)b * a.out_stride + (size_t)h * a.out_dim + d] = from_f<T>(o / L);
        else a.partial[(((size_t)b * a.heads + h) * a.n_splits + split) * (C + 2) + d] = o;
    }
    if (a.n_splits > 1 && threadIdx.x == 0) {
        float* p = a.partial + (((size_t)b * a.heads + h) * a.n_splits + split) * (C + 2);
        p[C] = M; p[C + 1] = L;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) latent_combine_kernel(LatentDecodeArgs a) {
    pdl_launch_dependents();
    __shared__ float f_s[128];                           // e^(m_s - M) of up to 128 splits at a time
    __shared__ float M_s, L_s;
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, C = a.C, n = a.n_splits;
    const float* p = a.partial + ((size_t)b * a.heads + h) * n * (C + 2);
    const float sink = (a.sink != nullptr) ? a.sink[h] : -INFINITY;
    if (threadIdx.x < 32) {
        float m = sink;
        for (int s = threadIdx.x; s < n; s += 32) m = fmaxf(m, p[(size_t)s * (C + 2) + C]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = threadIdx.x; s < n; s += 32) {
            const float ms = p[(size_t)s * (C + 2) + C];
            if (ms != -INFINITY) l += p[(size_t)s * (C + 2) + C + 1] * expf(ms - m);
        }
        l = warp_sum(l);
        if (threadIdx.x == 0) { M_s = m; L_s = l + ((sink != -INFINITY) ? expf(sink - m) : 0.f); }
    }
    __syncthreads();
    const float M = M_s, inv = 1.f / L_s;
    float o[4] = {0.f, 0.f, 0.f, 0.f};                   // columns threadIdx.x + 128 k (C <= 512)
    for (int s0 = 0; s0 < n; s0 += 128) {
        const int ns = min(128, n - s0);
        __syncthreads();
        if (threadIdx.x < ns) {
            const float ms = p[(size_t)(s0 + threadIdx.x) * (C + 2) + C];
            f_s[threadIdx.x] = (ms != -INFINITY) ? expf(ms - M) : 0.f;
        }
        __syncthreads();
        for (int s = 0; s < ns; s++) {
            const float f = f_s[s];
            const float* ps = p + (size_t)(s0 + s) * (C + 2);
#pragma unroll
            for (int k = 0; k < 4; k++) { const int d = threadIdx.x + 128 * k; if (d < C) o[k] = fmaf(ps[d], f, o[k]); }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int d = threadIdx.x + 128 * k;
        if (d < C) ((T*)a.out)[(size_t)b * a.out_stride + (size_t)h * a.out_dim + d] = from_f<T>(o[k] * inv);
    }
}

// ---------------------------------------------------------------------------
// The same decode on tensor cores (bfloat16): one CTA takes up to 16 heads of a sequence and a range of its
// keys, so that a cached row is fetched once for all of them.  Rows arrive 32 at a time (half a page, one
// contiguous piece of memory) by cp.async into a two-stage ring; S = Q' K^T with the heads as the 16
// rows of mma.sync m16n8k16 (each warp 8 of the 32 keys), the softmax of a head's 32 scores by one warp (four heads
// each), then O += P C with every warp taking a share of the latent's columns.  Partial (max, sum, o) go to the
// scratch that latent_combine_kernel folds (it also adds the sink).
// ---------------------------------------------------------------------------
constexpr int LD_BN = 32;

__device__ __forceinline__ uint32_t ld_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ld_cp16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ld_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ld_ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ld_ldsm2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ld_ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ld_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MT: tiles of 16 heads per CTA (1 or 2), with 4 * MT warps.  NP: pairs of 8-column tiles of the latent per warp
// (C <= NP * 16 * warps).  A warp scores 8 keys for 16 heads (four sums side by side, so that no product waits for the
// one before it), takes the softmax of four heads, and adds its share of the latent's columns for all heads.
template <int NP, int MT>
__global__ void __launch_bounds__(MT * 128) latent_decode_mma_kernel(LatentDecodeArgs a) {
    pdl_launch_dependents();
    constexpr int WARPS = 4 * MT, HEADS = 16 * MT, THREADS = WARPS * 32;
    extern __shared__ __align__(16) unsigned char sm[];
    const int KD = a.C + a.R, C = a.C;
    const int pitch = KD * 2 + 16;
    constexpr int PP = LD_BN * 2 + 16;
    unsigned char* q_s = sm;                                        // [HEADS][pitch]
    unsigned char* k_s = q_s + HEADS * pitch;                       // [2][LD_BN][pitch]
    float* s_s = (float*)(k_s + 2 * LD_BN * pitch);                 // [HEADS][LD_BN]
    unsigned char* p_s = (unsigned char*)(s_s + HEADS * LD_BN);     // [HEADS][PP]
    float* corr_s = (float*)(p_s + HEADS * PP);                     // [HEADS]
    const int b = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = hg * HEADS, nh = min(HEADS, a.heads - h0);
    pdl_wait();
    const int len = a.len_after[b];
    const int lo = latent_first_key(a.window, len), lo32 = lo / LD_BN * LD_BN;
    int per = (len - lo32 + a.n_splits - 1) / a.n_splits;
    per = (per + LD_BN - 1) / LD_BN * LD_BN;
    const int beg = lo32 + split * per, end = min(len, beg + per);
    const int* pt = a.page_table + (size_t)b * a.pt_stride;
    const bf16* pool = (const bf16*)a.pool;
    const int chunks = KD / 8;                                      // 16-byte pieces of a row
    auto load = [&](int stage, int j0) {
        const int r0 = a.ring_rows > 0 ? j0 % a.ring_rows : j0;       // 32 rows that start at a multiple of 32 lie in one page
        const bf16* src = pool + ((size_t)pt[r0 / a.page_rows] * a.page_rows + (r0 % a.page_rows)) * KD;
        unsigned char* dst = k_s + (size_t)stage * LD_BN * pitch;
        for (int c = threadIdx.x; c < LD_BN * chunks; c += THREADS) {
            const int r = c / chunks, ch = c % chunks;
            ld_cp16(dst + r * pitch + ch * 16, src + (size_t)r * KD + ch * 8, j0 + r < end && j0 + r >= lo);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (beg < end) load(0, beg);
    {   // the queries of this CTA's heads (rows past the last head: zeros)
        const bf16* q = (const bf16*)a.q + (size_t)b * a.q_stride + (size_t)h0 * KD;
        for (int c = threadIdx.x; c < HEADS * chunks; c += THREADS) {
            const int r = c / chunks, ch = c % chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < nh) v = *(const uint4*)(q + (size_t)r * KD + ch * 8);
            *(uint4*)(q_s + r * pitch + ch * 16) = v;
        }
    }
    float o[MT][NP * 2][4];
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int n = 0; n < NP * 2; n++) { o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.f; }
    float m_run[4], l_run[4];                                       // of heads 4 * warp + i (every lane holds a copy)
#pragma unroll
    for (int i = 0; i < 4; i++) { m_run[i] = -INFINITY; l_run[i] = 0.f; }
    const int sm_tile = warp / 4, sn_tile = warp % 4;               // scores: this warp's 16 heads and 8 keys
    const int n_tiles = beg < end ? (end - beg + LD_BN - 1) / LD_BN : 0;
    for (int it = 0; it < n_tiles; it++) {
        const int j0 = beg + it * LD_BN;
        if (it + 1 < n_tiles) { load((it + 1) & 1, j0 + LD_BN); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const unsigned char* kt = k_s + (size_t)(it & 1) * LD_BN * pitch;
        // ---- scores
        float sc[4][4];
#pragma unroll
        for (int u = 0; u < 4; u++) { sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.f; }
        const uint32_t qa = ld_smem(q_s + (sm_tile * 16 + (lane & 15)) * pitch + (lane >> 4) * 16);
        const uint32_t ka = ld_smem(kt + (sn_tile * 8 + (lane & 7)) * pitch + ((lane >> 3) & 1) * 16);
        const int ksteps = KD / 16;
        for (int ks = 0; ks < ksteps; ks += 4) {
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (ks + u < ksteps) {
                    uint32_t fa[4], b0, b1;
                    ld_ldsm4(qa + (ks + u) * 32, fa[0], fa[1], fa[2], fa[3]);
                    ld_ldsm2(ka + (ks + u) * 32, b0, b1);
                    ld_mma(sc[u], fa, b0, b1);
                }
            }
        }
        {
            const int r = sm_tile * 16 + (lane >> 2), cc = sn_tile * 8 + (lane & 3) * 2;
            s_s[r * LD_BN + cc] = (sc[0][0] + sc[1][0] + sc[2][0] + sc[3][0]) * a.scale;
            s_s[r * LD_BN + cc + 1] = (sc[0][1] + sc[1][1] + sc[2][1] + sc[3][1]) * a.scale;
            s_s[(r + 8) * LD_BN + cc] = (sc[0][2] + sc[1][2] + sc[2][2] + sc[3][2]) * a.scale;
            s_s[(r + 8) * LD_BN + cc + 1] = (sc[0][3] + sc[1][3] + sc[2][3] + sc[3][3]) * a.scale;
        }
        __syncthreads();
        // ---- softmax of four heads per warp over the tile's 32 keys (one key per lane)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = warp * 4 + i;
            const float v = (j0 + lane < end && j0 + lane >= lo) ? s_s[r * LD_BN + lane] : -INFINITY;
            const float mn = fmaxf(m_run[i], warp_max(v));
            const float corr = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - mn);
            const float p = (v == -INFINITY) ? 0.f : expf(v - mn);
            l_run[i] = l_run[i] * corr + warp_sum(p);
            m_run[i] = mn;
            *(bf16*)(p_s + r * PP + lane * 2) = __float2bfloat16_rn(p);
            if (lane == 0) corr_s[r] = corr;
        }
        __syncthreads();
        // ---- O = O * corr + P C, this warp's share of the latent's columns, for every tile of heads
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float ca = corr_s[m * 16 + (lane >> 2)], cb = corr_s[m * 16 + (lane >> 2) + 8];
            uint32_t pa[LD_BN / 16][4];
#pragma unroll
            for (int kk = 0; kk < LD_BN / 16; kk++)
                ld_ldsm4(ld_smem(p_s + (m * 16 + (lane & 15)) * PP + (kk * 16 + (lane >> 4) * 8) * 2), pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3]);
#pragma unroll
            for (int j = 0; j < NP; j++) {
                const int col0 = (j * WARPS + warp) * 16;
                if (col0 >= C) continue;
                float* oa = o[m][2 * j]; float* ob = o[m][2 * j + 1];
                oa[0] *= ca; oa[1] *= ca; oa[2] *= cb; oa[3] *= cb; ob[0] *= ca; ob[1] *= ca; ob[2] *= cb; ob[3] *= cb;
#pragma unroll
                for (int kk = 0; kk < LD_BN / 16; kk++) {
                    uint32_t b0, b1, b2, b3;
                    ld_ldsm4_t(ld_smem(kt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * pitch + (col0 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                    ld_mma(oa, pa[kk], b0, b1);
                    ld_mma(ob, pa[kk], b2, b3);
                }
            }
        }
        __syncthreads();                                            // the load after next overwrites this stage; s_s and p_s are free
    }
    // ---- partial results: [b][h][split][C + 2]
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const int ra = m * 16 + (lane >> 2), rb = ra + 8;
#pragma unroll
        for (int j = 0; j < NP; j++) {
            const int col0 = (j * WARPS + warp) * 16;
            if (col0 >= C) continue;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int col = col0 + half * 8 + (lane & 3) * 2;
                const float* acc = o[m][2 * j + half];
                if (ra < nh) { float* p = a.partial + (((size_t)b * a.heads + h0 + ra) * a.n_splits + split) * (C + 2); p[col] = acc[0]; p[col + 1] = acc[1]; }
                if (rb < nh) { float* p = a.partial + (((size_t)b * a.heads + h0 + rb) * a.n_splits + split) * (C + 2); p[col] = acc[2]; p[col + 1] = acc[3]; }
            }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = warp * 4 + i;
            if (r < nh) { float* p = a.partial + (((size_t)b * a.heads + h0 + r) * a.n_splits + split) * (C + 2); p[C] = m_run[i]; p[C + 1] = l_run[i]; }
        }
    }
}

extern "C" int tb_latent_decode_mma_takes(int C, int R) {
    return C > 0 && C % 16 == 0 && (C + R) % 16 == 0 && C <= 512 && (C + R) <= 1024;
}

extern "C" int tb_latent_decode_mma(const LatentDecodeArgs* args, int batch, cudaStream_t stream) {
    if (batch <= 0) return 0;
    const LatentDecodeArgs& a = *args;
    if (!tb_latent_decode_mma_takes(a.C, a.R)) return tb_refuse("latent_decode_mma: C=%d R=%d (multiples of 16, C <= 512)", a.C, a.R);
    if (a.partial == nullptr || a.n_splits < 1 || a.n_splits > 65535 || a.out_dim < a.C || a.page_rows % LD_BN)
        return tb_refuse("latent_decode_mma: n_splits=%d needs scratch; pages of %d rows", a.n_splits, a.page_rows);
    if (((uintptr_t)a.q & 15) || (a.q_stride % 8) || ((uintptr_t)a.pool & 15)) return tb_refuse("latent_decode_mma: rows must be 16-byte aligned");
    const int KD = a.C + a.R, pitch = KD * 2 + 16;
    const int mt = a.heads > 16 ? 2 : 1, heads_cta = 16 * mt, warps = 4 * mt;
    const size_t smem = (size_t)heads_cta * pitch + 2 * (size_t)LD_BN * pitch + heads_cta * LD_BN * 4 + heads_cta * (LD_BN * 2 + 16) + heads_cta * 4;
    const int np = (a.C + 16 * warps - 1) / (16 * warps);
    dim3 grid(batch, (a.heads + heads_cta - 1) / heads_cta, a.n_splits);
#define LD_MMA(N, M) do { \
        static bool set = false; \
        if (!set) { cudaError_t e = cudaFuncSetAttribute(latent_decode_mma_kernel<N, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
                    if (e != cudaSuccess) return (int)e; set = true; } \
        tb_launch(latent_decode_mma_kernel<N, M>, dim3(grid), dim3(warps * 32), smem, stream, a); } while (0)
    if (mt == 1) { if (np <= 2) LD_MMA(2, 1); else if (np <= 4) LD_MMA(4, 1); else LD_MMA(8, 1); }
    else { if (np <= 1) LD_MMA(1, 2); else if (np <= 2) LD_MMA(2, 2); else LD_MMA(4, 2); }
    int st = tb_launch_status();
    if (st) return st;
    tb_launch(latent_combine_kernel<bf16>, dim3(batch, a.heads), dim3(128), 0, stream, a);
    return tb_launch_status();
}

extern "C" int tb_latent_decode(const LatentDecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    if (batch <= 0) return 0;
    const LatentDecodeArgs& a = *args;
    if (a.heads <= 0 || a.heads > 65535 || a.C <= 0 || a.R < 0 || a.C > 512 || a.out_dim < a.C)
        return tb_refuse("latent_decode: heads=%d C=%d R=%d out_dim=%d (C at most 512)", a.heads, a.C, a.R, a.out_dim);
    if (a.n_splits < 1 || a.n_splits > 65535 || (a.n_splits > 1 && a.partial == nullptr))
        return tb_refuse("latent_decode: n_splits=%d needs scratch", a.n_splits);
    const int warps = 4;
    const size_t smem = ((size_t)(a.C + a.R) + (size_t)warps * (a.C + 2)) * sizeof(float);
    int nc = 1;
    while (nc * 32 < a.C) nc <<= 1;
    dim3 grid(batch, a.heads, a.n_splits);
#define LAT_DEC(N) TB_DISPATCH_1(dtype, T, tb_launch(latent_decode_kernel<T, N>, dim3(grid), dim3(warps * 32), smem, stream, a))
    switch (nc) {
    case 1: LAT_DEC(1); break;
    case 2: LAT_DEC(2); break;
    case 4: LAT_DEC(4); break;
    case 8: LAT_DEC(8); break;
    default: LAT_DEC(16); break;
    }
    int st = tb_launch_status();
    if (st || a.n_splits == 1) return st;
    TB_DISPATCH_1(dtype, T, tb_launch(latent_combine_kernel<T>, dim3(batch, a.heads), dim3(128), 0, stream, a));
    return tb_launch_status();
}
