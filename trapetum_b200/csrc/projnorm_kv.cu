// From the q/k/v(/gate) product to what the attention kernels read, for mixers that norm q and k over the WHOLE
// projection (all heads at once) before the rotation, weigh each head's scores with a number of its own, have values
// of another size than the keys, and gate each head's output.
//
// The input is the product as 32-bit partial sums [splits][tokens][in_width] (added here in split order) with the
// columns [q: H x dim | k: G x dim | v: G x vdim | gate: H].  Per token, all in 32-bit, rounded once on the way out:
//
//   q <- q / sqrt(mean(q^2) + eps) * wq          mean over all H x dim numbers; wq of that size   (if wq is given)
//   k <- k / sqrt(mean(k^2) + eps) * wk          mean over all G x dim numbers                    (if wk is given)
//   q_h <- q_h * head_scale[h]                   (if given; the score is linear in q, so this weighs head h's scores)
//   the first R dims of every q and k head turned by pos * inv_freq[i], pair (i, i + R/2)         (if R > 0)
//   gate_out[t][h] = sigmoid(gate column h)      (if asked for)
//
// The output row is [q heads | k heads | v heads], every head padded with zeros to D numbers (D >= dim, vdim: one
// head size for keys and values, which is what the cache and the attention kernels take; zeros change neither a
// score nor the part of the output that is kept); k and v also go to the cache line (row = ring_rows ? pos %
// ring_rows : pos, page = page_table[seq, row / page_rows]; in a ring only tokens with pos >= len_after - ring_rows
// are written).
//
// A bias (one 32-bit number per column of the product) is added to the summed row first, if given.
//
// tb_head_gate multiplies every head of an attention output [tokens][H x D] by its token's gate, in place.
//
// tb_head_difference folds an attention output whose heads come in pairs (two score maps over the same values):
// o = a1 - lam * a2 over the head's first vdim numbers, o / sqrt(mean(o^2) + eps) * out_scale, zeros in the padding.
//
// One CTA per token (256 threads, 1,024 when the tokens are few); the token's summed row lies in shared memory.
#include "common.cuh"

TB_EXPORT_ERROR()

struct ProjNormKvArgs {
    const float* partial; int n_splits; long long split_stride, partial_row_stride;
    void* out; long long out_row_stride;          // [tokens][(H + 2 G) * D]
    float* gate_out;                              // [tokens][H] or null
    int n_heads, n_kv_heads, dim, vdim, D;
    const float* q_norm_w; const float* k_norm_w; // [H * dim], [G * dim] or null
    float eps;
    const float* head_scale;                      // [H] or null
    int rotary_dim; const float* inv_freq;        // [rotary_dim / 2]
    const int* positions; const int* token_seq; const int* len_after;
    void* k_pool; void* v_pool; const int* page_table; int pt_stride; int page_rows; int ring_rows;
    const float* bias;                            // [in_width rounded up to 4] added to the summed row, or null
};

// Eight (four) consecutive numbers of an output row, rounded and stored with one or two wide stores.
template <typename T> __device__ __forceinline__ void store8(T* dst, const float (&y)[8]);
template <> __device__ __forceinline__ void store8<float>(float* dst, const float (&y)[8]) {
    ((float4*)dst)[0] = make_float4(y[0], y[1], y[2], y[3]);
    ((float4*)dst)[1] = make_float4(y[4], y[5], y[6], y[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* dst, const float (&y)[8]) {
    union { uint4 u; __nv_bfloat162 h[4]; } v;
#pragma unroll
    for (int j = 0; j < 4; j++) v.h[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
    *(uint4*)dst = v.u;
}
template <typename T> __device__ __forceinline__ void store4(T* dst, const float4& y);
template <> __device__ __forceinline__ void store4<float>(float* dst, const float4& y) { *(float4*)dst = y; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* dst, const float4& y) {
    union { uint2 u; __nv_bfloat162 h[2]; } v;
    v.h[0] = __floats2bfloat162_rn(y.x, y.y);
    v.h[1] = __floats2bfloat162_rn(y.z, y.w);
    *(uint2*)dst = v.u;
}

// MODE 1 and 2: every head size involved (dim, vdim, D, half of the rotated part) is a multiple of 4 and the rows are
// 16-byte aligned, so the partial sums are read 16 bytes at a time and a thread makes four numbers of the output at a
// time: a warp's 16-byte reads of the row in shared memory then touch every bank once (eight numbers a thread, read one
// by one, met the same bank eight times and made the kernel wait on shared memory).  MODE 2: the pieces of a head
// divide the block's threads (heads padded to 64, 128 or 256), so a thread keeps its place in the head and walks the
// heads: no division per piece, its cosines and sines fetched once, and the loads of consecutive heads' norm weights
// do not wait for one another.  MODE 0: any sizes, number by number.
template <typename T, int MODE>
__global__ void __launch_bounds__(1024) projnorm_kv_kernel(ProjNormKvArgs a) {
    constexpr bool VEC = MODE != 0;
    pdl_launch_dependents();
    extern __shared__ __align__(16) float row[];          // [in_width rounded up to 4] then cos[half], sin[half]
    __shared__ float red[64];
    const int t = blockIdx.x;
    const int H = a.n_heads, G = a.n_kv_heads, dim = a.dim, vdim = a.vdim, D = a.D;
    const int nq = H * dim, nk = G * dim, nv = G * vdim;
    const int in_width = nq + nk + nv + (a.gate_out != nullptr ? H : 0);
    const int R = a.rotary_dim, half = R >> 1;
    float* cs = row + ((in_width + 3) & ~3);
    float* sn = cs + half;
    pdl_wait();
    const int pos = a.positions[t];
    const int b = a.k_pool != nullptr ? a.token_seq[t] : 0;
    const float* src = a.partial + (size_t)t * a.partial_row_stride;
    float ssq = 0.f, ssk = 0.f;                           // this thread's share of the sums of squares of q and of k
    if (VEC) {
        // 16 bytes of every split in flight together, summed in split order in registers; nq and nk are multiples of
        // eight here, so a piece lies in q, in k or behind them
        const int n4 = (in_width + 3) >> 2;               // the product's rows are padded to whole 16-byte pieces
        const int q4 = nq >> 2, k4 = (nq + nk) >> 2;
        float4* row4 = (float4*)row;
        const float4* s4 = (const float4*)src;
        const size_t st4 = (size_t)a.split_stride >> 2;
        if (a.n_splits == 1) {
            // a prompt's product comes whole: four pieces of the row in flight per thread
#pragma unroll 4
            for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                float4 r = __ldg(s4 + i);
                if (a.bias != nullptr) { const float4 bb = __ldg((const float4*)a.bias + i); r.x += bb.x; r.y += bb.y; r.z += bb.z; r.w += bb.w; }
                row4[i] = r;
                const float s2 = r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
                if (i < q4) ssq += s2; else if (i < k4) ssk += s2;
            }
        } else {
#pragma unroll 2
            for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                float4 r = __ldg(s4 + i);
#pragma unroll 8
                for (int sp = 1; sp < a.n_splits; sp++) {
                    const float4 v = __ldg(s4 + sp * st4 + i);
                    r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;
                }
                if (a.bias != nullptr) { const float4 bb = __ldg((const float4*)a.bias + i); r.x += bb.x; r.y += bb.y; r.z += bb.z; r.w += bb.w; }
                row4[i] = r;
                const float s2 = r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
                if (i < q4) ssq += s2; else if (i < k4) ssk += s2;
            }
        }
    } else {
        for (int i = threadIdx.x; i < in_width; i += blockDim.x) {
            float s = 0.f;
            for (int sp = 0; sp < a.n_splits; sp++) s += src[(size_t)sp * a.split_stride + i];       // in split order
            if (a.bias != nullptr) s += a.bias[i];
            row[i] = s;
            if (i < nq) ssq += s * s; else if (i < nq + nk) ssk += s * s;
        }
    }
    // the angles of this token's position: once per token, not once per head
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * a.inv_freq[i], &sn[i], &cs[i]);
    // where this token's k and v go in the cache (if anywhere); these dependent loads follow the row's, whose wait
    // has covered the position's and the sequence's
    bool store = false;
    size_t cache_row = 0;
    if (a.k_pool != nullptr) {
        store = true;
        int r = pos;
        if (a.ring_rows > 0) { store = pos >= a.len_after[b] - a.ring_rows; r = pos % a.ring_rows; }
        if (store) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            cache_row = (size_t)page * G * a.page_rows + (r % a.page_rows);          // + kv head * page_rows, then * D
        }
    }
    // both sums in one pass over the block (its first barrier also publishes the row and the angles)
    float rq = 1.f, rk = 1.f;
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
        ssq = warp_sum(ssq); ssk = warp_sum(ssk);
        if (lane == 0) { red[warp] = ssq; red[32 + warp] = ssk; }
        __syncthreads();
        float tq = lane < nwarp ? red[lane] : 0.f, tk = lane < nwarp ? red[32 + lane] : 0.f;
        tq = warp_sum(tq); tk = warp_sum(tk);
        if (a.q_norm_w != nullptr) rq = 1.0f / sqrtf(tq / (float)nq + a.eps);
        if (a.k_norm_w != nullptr) rk = 1.0f / sqrtf(tk / (float)nk + a.eps);
    }
    T* orow = (T*)a.out + (size_t)t * a.out_row_stride;
    const int n_qk = (H + G) * D;
    T* vrow = orow + n_qk;
    if (VEC) {
        const int per = D >> 2;                                                      // pieces of four per head
        const int hstep = MODE == 2 ? blockDim.x / per : 0;
        int hs = MODE == 2 ? threadIdx.x / per : 0, i0 = MODE == 2 ? (threadIdx.x - hs * per) << 2 : 0;
#pragma unroll 2
        for (int u = threadIdx.x; u < (H + G) * per; u += blockDim.x) {
            if (MODE != 2) { hs = u / per; i0 = (u - hs * per) << 2; }
            const bool is_q = hs < H;
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i0 < dim) {
                const int head = is_q ? hs : hs - H;
                const int c0 = head * dim;
                const float* x = row + (is_q ? 0 : nq) + c0;
                const float* w = is_q ? a.q_norm_w : a.k_norm_w;
                const float f = (is_q ? rq : rk) * ((is_q && a.head_scale != nullptr) ? a.head_scale[head] : 1.f);
                float4 xi = *(const float4*)(x + i0);
                xi.x *= f; xi.y *= f; xi.z *= f; xi.w *= f;
                if (w != nullptr) {
                    const float4 wi = __ldg((const float4*)(w + c0 + i0));
                    xi.x *= wi.x; xi.y *= wi.y; xi.z *= wi.z; xi.w *= wi.w;
                }
                if (i0 < R) {
                    const bool lo = i0 < half;
                    const int j0 = lo ? i0 + half : i0 - half, a0 = lo ? i0 : i0 - half;
                    float4 xj = *(const float4*)(x + j0);
                    xj.x *= f; xj.y *= f; xj.z *= f; xj.w *= f;
                    if (w != nullptr) {
                        const float4 wj = __ldg((const float4*)(w + c0 + j0));
                        xj.x *= wj.x; xj.y *= wj.y; xj.z *= wj.z; xj.w *= wj.w;
                    }
                    const float4 c = *(const float4*)(cs + a0), sv = *(const float4*)(sn + a0);
                    const float sg = lo ? -1.f : 1.f;
                    y.x = xi.x * c.x + sg * (xj.x * sv.x); y.y = xi.y * c.y + sg * (xj.y * sv.y);
                    y.z = xi.z * c.z + sg * (xj.z * sv.z); y.w = xi.w * c.w + sg * (xj.w * sv.w);
                } else {
                    y = xi;
                }
            }
            store4<T>(orow + (size_t)hs * D + i0, y);
            if (!is_q && store) store4<T>((T*)a.k_pool + (cache_row + (size_t)(hs - H) * a.page_rows) * D + i0, y);
            if (MODE == 2) hs += hstep;
        }
        for (int u = threadIdx.x; u < G * per; u += blockDim.x) {
            const int g = u / per, i0 = (u - g * per) << 2;
            const float4 y = i0 < vdim ? *(const float4*)(row + nq + nk + g * vdim + i0) : make_float4(0.f, 0.f, 0.f, 0.f);
            store4<T>(vrow + (size_t)g * D + i0, y);
            if (store) store4<T>((T*)a.v_pool + (cache_row + (size_t)g * a.page_rows) * D + i0, y);
        }
    } else {
        // q and k heads: normed, weighed, rotated, padded
        for (int e = threadIdx.x; e < n_qk; e += blockDim.x) {
            const int hs = e / D, i = e - hs * D;
            const bool is_q = hs < H;
            float y = 0.f;
            if (i < dim) {
                const int head = is_q ? hs : hs - H;
                const int c0 = head * dim;                                               // the head's first column in its projection
                const float* x = row + (is_q ? 0 : nq);
                const float* w = is_q ? a.q_norm_w : a.k_norm_w;
                const float f = (is_q ? rq : rk) * ((is_q && a.head_scale != nullptr) ? a.head_scale[head] : 1.f);
                const float xi = x[c0 + i] * (w != nullptr ? w[c0 + i] : 1.f) * f;
                if (i < R) {
                    const int j = i < half ? i + half : i - half, ai = i < half ? i : i - half;
                    const float xj = x[c0 + j] * (w != nullptr ? w[c0 + j] : 1.f) * f;
                    y = i < half ? xi * cs[ai] - xj * sn[ai] : xi * cs[ai] + xj * sn[ai];
                } else {
                    y = xi;
                }
            }
            const T yy = from_f<T>(y);
            orow[e] = yy;
            if (!is_q && store) ((T*)a.k_pool)[(cache_row + (size_t)(hs - H) * a.page_rows) * D + i] = yy;
        }
        // v heads: as they are, padded
        for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
            const int g = e / D, i = e - g * D;
            const T yy = from_f<T>(i < vdim ? row[nq + nk + g * vdim + i] : 0.f);
            vrow[e] = yy;
            if (store) ((T*)a.v_pool)[(cache_row + (size_t)g * a.page_rows) * D + i] = yy;
        }
    }
    if (a.gate_out != nullptr)
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            a.gate_out[(size_t)t * H + h] = 1.f / (1.f + expf(-row[nq + nk + nv + h]));
}

extern "C" int tb_projnorm_kv(const ProjNormKvArgs* args, int out_dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    ProjNormKvArgs a = *args;
    if (a.n_heads <= 0 || a.n_kv_heads < 0 || a.dim <= 0 || a.vdim <= 0 || a.D < a.dim || a.D < a.vdim)
        return tb_refuse("projnorm_kv: heads=%d kv heads=%d dim=%d vdim=%d padded to %d", a.n_heads, a.n_kv_heads, a.dim, a.vdim, a.D);
    if (a.partial == nullptr || a.n_splits < 1) return tb_refuse("projnorm_kv: needs the product's partial sums");
    if (a.rotary_dim < 0 || a.rotary_dim % 2 || a.rotary_dim > a.dim || (a.rotary_dim > 0 && a.inv_freq == nullptr))
        return tb_refuse("projnorm_kv: rotary_dim=%d must be even, at most dim=%d, and come with its table", a.rotary_dim, a.dim);
    if (a.k_pool != nullptr && (a.page_rows <= 0 || a.page_table == nullptr || a.v_pool == nullptr))
        return tb_refuse("projnorm_kv: a cache write needs page_rows > 0, a page table and both pools");
    if (a.ring_rows > 0 && a.ring_rows % a.page_rows != 0)
        return tb_refuse("projnorm_kv: ring_rows=%d must be a multiple of page_rows=%d", a.ring_rows, a.page_rows);
    const long long in_width = (long long)a.n_heads * a.dim + (long long)a.n_kv_heads * (a.dim + a.vdim) + (a.gate_out ? a.n_heads : 0);
    const size_t smem = (size_t)(((in_width + 3) & ~3LL) + a.rotary_dim) * sizeof(float);
    if (smem > 200 * 1024) return tb_refuse("projnorm_kv: a projection of %lld numbers exceeds one block's shared memory", in_width);
    const int half = a.rotary_dim / 2;
    const size_t el = out_dtype == TB_BF16 ? 2 : 4;
    const bool vec = a.dim % 4 == 0 && a.vdim % 4 == 0 && a.D % 4 == 0 && half % 4 == 0
        && ((uintptr_t)a.partial % 16 == 0) && a.split_stride % 4 == 0 && a.partial_row_stride % 4 == 0
        && a.partial_row_stride >= ((in_width + 3) & ~3LL)
        && ((uintptr_t)a.out % 16 == 0) && (a.out_row_stride * el) % 16 == 0
        && (a.q_norm_w == nullptr || (uintptr_t)a.q_norm_w % 16 == 0) && (a.k_norm_w == nullptr || (uintptr_t)a.k_norm_w % 16 == 0)
        && (a.k_pool == nullptr || ((uintptr_t)a.k_pool % 16 == 0 && (uintptr_t)a.v_pool % 16 == 0))
        && (a.bias == nullptr || (uintptr_t)a.bias % 16 == 0);
    // few tokens (a decode step) leave most of the GPU idle and are a chain of memory waits: four times the threads a
    // token shorten the chain; many tokens fill the GPU with blocks of 256
    const int threads = n_tokens <= 2 * 148 ? 1024 : 256;
    const int mode = !vec ? 0 : (256 % (a.D / 4) == 0 ? 2 : 1);
#define TB_PROJNORM_LAUNCH(T, V) do { \
        if (smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(projnorm_kv_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e; \
        } \
        tb_launch(projnorm_kv_kernel<T, V>, dim3(n_tokens), dim3(threads), smem, stream, a); } while (0)
#define TB_PROJNORM_MODES(T) do { if (mode == 2) TB_PROJNORM_LAUNCH(T, 2); else if (mode == 1) TB_PROJNORM_LAUNCH(T, 1); else TB_PROJNORM_LAUNCH(T, 0); } while (0)
    if (out_dtype == TB_BF16) TB_PROJNORM_MODES(bf16);
    else if (out_dtype == TB_F32) TB_PROJNORM_MODES(float);
    else return tb_refuse("projnorm_kv: output dtype %d", out_dtype);
#undef TB_PROJNORM_MODES
#undef TB_PROJNORM_LAUNCH
    return tb_launch_status();
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, const float* __restrict__ gate, long long n, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    o[i] = from_f<T>(to_f<T>(o[i]) * gate[i / D]);
}

// Eight numbers a thread (D a multiple of 8: a piece lies in one head), 16-byte loads and stores.
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ o, const float* __restrict__ gate, long long n8, int per) {
    pdl_launch_dependents();
    pdl_wait();
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n8) return;
    const float g = gate[u / per];
    T* p = o + u * 8;
    float y[8];
    if (sizeof(T) == 2) {
        union { uint4 u4; __nv_bfloat162 h[4]; } v;
        v.u4 = *(const uint4*)p;
#pragma unroll
        for (int j = 0; j < 4; j++) { const float2 f = __bfloat1622float2(v.h[j]); y[2 * j] = f.x * g; y[2 * j + 1] = f.y * g; }
    } else {
        const float4 a = ((const float4*)p)[0], b = ((const float4*)p)[1];
        y[0] = a.x * g; y[1] = a.y * g; y[2] = a.z * g; y[3] = a.w * g; y[4] = b.x * g; y[5] = b.y * g; y[6] = b.z * g; y[7] = b.w * g;
    }
    store8<T>(p, y);
}

// o [tokens][H * D] (contiguous) times gate [tokens][H], in place.
extern "C" int tb_head_gate(void* o, int dtype, const float* gate, int n_tokens, int n_heads, int D, cudaStream_t stream) {
    const long long n = (long long)n_tokens * n_heads * D;
    if (n <= 0) return 0;
    if (D % 8 == 0 && (uintptr_t)o % 16 == 0) {
        const long long n8 = n / 8;
        TB_DISPATCH_1(dtype, T, tb_launch(head_gate_vec_kernel<T>, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (T*)o, gate, n8, D / 8));
        return tb_launch_status();
    }
    TB_DISPATCH_1(dtype, T, tb_launch(head_gate_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (T*)o, gate, n, D));
    return tb_launch_status();
}

// One warp per (token, head): in [rows][2][D] -> out [rows][D], the difference and its unit norm in 32-bit.
template <typename T>
__global__ void head_difference_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, int D, int vdim,
                                       float lam, float eps, float out_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* a1 = in + r * 2 * D;
    const T* a2 = a1 + D;
    float sq = 0.f;
    for (int d = lane; d < vdim; d += 32) { const float o = to_f<T>(a1[d]) - lam * to_f<T>(a2[d]); sq = fmaf(o, o, sq); }
    const float f = out_scale / sqrtf(warp_sum(sq) / (float)vdim + eps);
    T* o_row = out + r * D;
    for (int d = lane; d < D; d += 32)
        o_row[d] = from_f<T>(d < vdim ? (to_f<T>(a1[d]) - lam * to_f<T>(a2[d])) * f : 0.f);
}

extern "C" int tb_head_difference(const void* in, void* out, int dtype, int n_tokens, int n_heads, int D, int vdim, float lam,
                                  float eps, float out_scale, cudaStream_t stream) {
    const long long rows = (long long)n_tokens * n_heads;
    if (rows <= 0) return 0;
    if (D <= 0 || vdim <= 0 || vdim > D) return tb_refuse("head_difference: D=%d vdim=%d", D, vdim);
    TB_DISPATCH_1(dtype, T, tb_launch(head_difference_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, stream,
                                      (const T*)in, (T*)out, rows, D, vdim, lam, eps, out_scale));
    return tb_launch_status();
}
