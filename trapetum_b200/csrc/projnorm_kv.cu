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
// tb_head_gate multiplies every head of an attention output [tokens][H x D] by its token's gate, in place.
//
// One CTA per token; the token's summed row lies in shared memory.
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
};

template <typename T>
__global__ void __launch_bounds__(256) projnorm_kv_kernel(ProjNormKvArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float row[];          // [in_width]
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int H = a.n_heads, G = a.n_kv_heads, dim = a.dim, vdim = a.vdim, D = a.D;
    const int nq = H * dim, nk = G * dim, nv = G * vdim;
    const int in_width = nq + nk + nv + (a.gate_out != nullptr ? H : 0);
    pdl_wait();
    const float* src = a.partial + (size_t)t * a.partial_row_stride;
    for (int i = threadIdx.x; i < in_width; i += blockDim.x) {
        float s = 0.f;
        for (int sp = 0; sp < a.n_splits; sp++) s += src[(size_t)sp * a.split_stride + i];       // in split order
        row[i] = s;
    }
    __syncthreads();
    float rq = 1.f, rk = 1.f;
    if (a.q_norm_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) ss += row[i] * row[i];
        rq = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
    }
    if (a.k_norm_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) ss += row[nq + i] * row[nq + i];
        rk = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
    }
    const int pos = a.positions[t];
    const int R = a.rotary_dim, half = R >> 1;
    // where this token's k and v go in the cache (if anywhere)
    bool store = false;
    size_t cache_row = 0;
    if (a.k_pool != nullptr) {
        const int b = a.token_seq[t];
        store = true;
        int r = pos;
        if (a.ring_rows > 0) { store = pos >= a.len_after[b] - a.ring_rows; r = pos % a.ring_rows; }
        if (store) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            cache_row = (size_t)page * G * a.page_rows + (r % a.page_rows);          // + kv head * page_rows, then * D
        }
    }
    T* orow = (T*)a.out + (size_t)t * a.out_row_stride;
    // q and k heads: normed, weighed, rotated, padded
    const int n_qk = (H + G) * D;
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
                const int j = i < half ? i + half : i - half;
                const float xj = x[c0 + j] * (w != nullptr ? w[c0 + j] : 1.f) * f;
                float sn, cs;
                sincosf((float)pos * a.inv_freq[i < half ? i : i - half], &sn, &cs);
                y = i < half ? xi * cs - xj * sn : xi * cs + xj * sn;
            } else {
                y = xi;
            }
        }
        const T yy = from_f<T>(y);
        orow[e] = yy;
        if (!is_q && store) ((T*)a.k_pool)[(cache_row + (size_t)(hs - H) * a.page_rows) * D + i] = yy;
    }
    // v heads: as they are, padded
    T* vrow = orow + n_qk;
    for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
        const int g = e / D, i = e - g * D;
        const T yy = from_f<T>(i < vdim ? row[nq + nk + g * vdim + i] : 0.f);
        vrow[e] = yy;
        if (store) ((T*)a.v_pool)[(cache_row + (size_t)g * a.page_rows) * D + i] = yy;
    }
    if (a.gate_out != nullptr)
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            a.gate_out[(size_t)t * H + h] = 1.f / (1.f + expf(-row[nq + nk + nv + h]));
}

extern "C" int tb_projnorm_kv(const ProjNormKvArgs* args, int out_dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    ProjNormKvArgs a = *args;
    if (a.n_heads <= 0 || a.n_kv_heads <= 0 || a.dim <= 0 || a.vdim <= 0 || a.D < a.dim || a.D < a.vdim)
        return tb_refuse("projnorm_kv: heads=%d kv heads=%d dim=%d vdim=%d padded to %d", a.n_heads, a.n_kv_heads, a.dim, a.vdim, a.D);
    if (a.partial == nullptr || a.n_splits < 1) return tb_refuse("projnorm_kv: needs the product's partial sums");
    if (a.rotary_dim < 0 || a.rotary_dim % 2 || a.rotary_dim > a.dim || (a.rotary_dim > 0 && a.inv_freq == nullptr))
        return tb_refuse("projnorm_kv: rotary_dim=%d must be even, at most dim=%d, and come with its table", a.rotary_dim, a.dim);
    if (a.k_pool != nullptr && (a.page_rows <= 0 || a.page_table == nullptr || a.v_pool == nullptr))
        return tb_refuse("projnorm_kv: a cache write needs page_rows > 0, a page table and both pools");
    if (a.ring_rows > 0 && a.ring_rows % a.page_rows != 0)
        return tb_refuse("projnorm_kv: ring_rows=%d must be a multiple of page_rows=%d", a.ring_rows, a.page_rows);
    const long long in_width = (long long)a.n_heads * a.dim + (long long)a.n_kv_heads * (a.dim + a.vdim) + (a.gate_out ? a.n_heads : 0);
    const size_t smem = (size_t)in_width * sizeof(float);
    if (smem > 200 * 1024) return tb_refuse("projnorm_kv: a projection of %lld numbers exceeds one block's shared memory", in_width);
    if (smem > 48 * 1024) {
        cudaError_t e = out_dtype == TB_BF16 ? cudaFuncSetAttribute(projnorm_kv_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                             : cudaFuncSetAttribute(projnorm_kv_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    TB_DISPATCH_1(out_dtype, T, tb_launch(projnorm_kv_kernel<T>, dim3(n_tokens), dim3(256), smem, stream, a));
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

// o [tokens][H * D] (contiguous) times gate [tokens][H], in place.
extern "C" int tb_head_gate(void* o, int dtype, const float* gate, int n_tokens, int n_heads, int D, cudaStream_t stream) {
    const long long n = (long long)n_tokens * n_heads * D;
    if (n <= 0) return 0;
    TB_DISPATCH_1(dtype, T, tb_launch(head_gate_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (T*)o, gate, n, D));
    return tb_launch_status();
}
