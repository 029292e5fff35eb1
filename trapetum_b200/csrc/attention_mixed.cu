// Attention whose heads' scores are mixed before the softmax, for any head size, on the 32-bit FMA pipe.
//
// Per query i, key j and head h (query head g reads kv head g / (H / G)):
//   r_g  = q_g(i) . k_g(j)                                   every head's raw score
//   s_h  = sum_g mix[h][g] r_g                               mix: [H][H] 32-bit numbers; the caller folds the score's
//                                                            scale and a number per head into it
//   seen(i, j): j <= i, and  window > 0: i - j < window;  window < 0: i and j lie in the same block of -window
//               positions, blocks counted from position 0;  window == 0: nothing more
//   p_h  = exp(s_h) / (unit_sink + sum over seen j of exp(s_h))    unit_sink 1: the denominator also holds exp(0),
//                                                                  a sink without a key and without a value
//   o_h  = sum_j p_h(j) v_h(j)
// Because s_h needs every head's r of the same (i, j), one CTA takes all heads of a query: warp g makes r_g for 32
// keys (a key a lane), the warps exchange them through shared memory, warp h mixes its own s_h, keeps the running
// softmax and adds p.v with a slice of the head's dims per lane.  Dot products, mixing, softmax and the weighted sum
// are 32-bit for both dtypes.
//
//   tb_attn_mixed_prefill   queries and keys are the step's own packed tokens
//   tb_attn_mixed_decode    one query per sequence, keys from the paged cache (a ring if ring_rows > 0), the key range
//                           cut into pieces; partial (max, sum, o) per piece are folded in piece order
#include "common.cuh"

TB_EXPORT_ERROR()

struct MixedAttnArgs {
    const void* q; long long q_stride;                    // [tokens] rows of H * D
    const void* k; const void* v; long long kv_stride;    // prefill: [tokens] rows of G * D; decode: pools [pages][G][page_rows][D]
    const int* seq_start; const int* token_seq;           // prefill: [batch + 1], [tokens]
    const int* page_table; int pt_stride; int page_rows; int ring_rows;
    const int* len_after;                                 // decode: [batch] keys in the cache, the new token included
    void* out; long long out_stride;                      // [tokens] rows of H * D
    const float* mix;                                     // [H][H]
    float* partial;                                       // decode: [batch][H][pieces][D + 2] when pieces > 1
    int H, G, D, n_tokens, window, unit_sink, n_pieces;
};

template <int NC>
struct MixAcc {
    float m, l, o[NC];
    __device__ void init() {
        m = -INFINITY; l = 0.f;
#pragma unroll
        for (int c = 0; c < NC; c++) o[c] = 0.f;
    }
};

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q_s, const T* __restrict__ krow, int D, bool vec) {
    float d = 0.f;
    constexpr int N = Vec<T>::N;
    if (vec) {
        for (int e = 0; e < D; e += N) {
            const uint4 u = *(const uint4*)(krow + e);
            const T* x = (const T*)&u;
#pragma unroll
            for (int i = 0; i < N; i++) d = fmaf(q_s[e + i], to_f<T>(x[i]), d);
        }
    } else {
        for (int e = 0; e < D; e++) d = fmaf(q_s[e], to_f<T>(krow[e]), d);
    }
    return d;
}

// 32 keys: lane `lane` of warp h holds key j0 + lane.  Every warp of the CTA calls this the same number of times.
template <typename T, int NC>
__device__ __forceinline__ void mixed_chunk(MixAcc<NC>& acc, const float* q_s, const float* mix_row, float* raw, int H, int h,
                                            const T* krow, const T* vrow, bool valid, int D, bool vec, int lane) {
    raw[h * 32 + lane] = valid ? dot_row<T>(q_s, krow, D, vec) : 0.f;
    __syncthreads();
    float s = -INFINITY;
    if (valid) {
        s = 0.f;
        for (int g = 0; g < H; g++) s = fmaf(mix_row[g], raw[g * 32 + lane], s);
    }
    const float cm = warp_max(s);
    if (cm == -INFINITY) return;
    const float m_new = fmaxf(acc.m, cm);
    const float corr = (acc.m == -INFINITY) ? 0.f : expf(acc.m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    acc.l = acc.l * corr + warp_sum(p);
    acc.m = m_new;
#pragma unroll
    for (int c = 0; c < NC; c++) acc.o[c] *= corr;
    for (int jj = 0; jj < 32; jj++) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)vrow, jj);
        if (pj == 0.f) continue;
        const T* v = (const T*)(uintptr_t)vp;
#pragma unroll
        for (int c = 0; c < NC; c++) {
            const int d = lane + 32 * c;
            if (d < D) acc.o[c] = fmaf(pj, to_f<T>(v[d]), acc.o[c]);
        }
    }
}

// The first position a query at position i sees (see the head of the file).
__device__ __forceinline__ int first_seen(int window, int i) {
    if (window > 0) return i - window + 1 > 0 ? i - window + 1 : 0;
    if (window < 0) return (i / (-window)) * (-window);
    return 0;
}

template <typename T, int NC>
__global__ void attn_mixed_prefill_kernel(MixedAttnArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int H = a.H, D = a.D;
    float* q_s = smem;                         // [H][D]
    float* mix_s = q_s + H * D;                // [H][H]
    float* raw = mix_s + H * H;                // [2][H][32]
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int kvh = h / (H / a.G);
    for (int e = threadIdx.x; e < H * H; e += blockDim.x) mix_s[e] = a.mix[e];
    pdl_wait();
    const int s0 = a.seq_start[a.token_seq[t]];
    const int i = t - s0;
    const T* qrow = (const T*)a.q + (size_t)t * a.q_stride;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) q_s[e] = to_f<T>(qrow[e]);
    __syncthreads();
    const bool vec = (D % Vec<T>::N) == 0 && (a.kv_stride % Vec<T>::N) == 0 && (((uintptr_t)a.k) & 15) == 0 && (((uintptr_t)a.v) & 15) == 0;
    MixAcc<NC> acc; acc.init();
    const int lo = first_seen(a.window, i);
    int buf = 0;
    for (int j0 = lo; j0 <= i; j0 += 32, buf ^= 1) {
        const int j = j0 + lane;
        const bool valid = j <= i;
        const size_t off = (size_t)(s0 + j) * a.kv_stride + (size_t)kvh * D;
        mixed_chunk<T, NC>(acc, q_s + h * D, mix_s + h * H, raw + buf * H * 32, H, h,
                           valid ? (const T*)a.k + off : nullptr, valid ? (const T*)a.v + off : nullptr, valid, D, vec, lane);
    }
    float inv = 1.f / acc.l;
    if (a.unit_sink) {
        const float M = fmaxf(acc.m, 0.f);
        const float f = expf(acc.m - M);
        inv = f / (acc.l * f + expf(-M));
    }
    T* orow = (T*)a.out + (size_t)t * a.out_stride + (size_t)h * D;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int d = lane + 32 * c;
        if (d < D) orow[d] = from_f<T>(acc.o[c] * inv);
    }
}

template <typename T, int NC>
__global__ void attn_mixed_decode_kernel(MixedAttnArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int H = a.H, D = a.D;
    float* q_s = smem;
    float* mix_s = q_s + H * D;
    float* raw = mix_s + H * H;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x, piece = blockIdx.y;
    const int kvh = h / (H / a.G);
    for (int e = threadIdx.x; e < H * H; e += blockDim.x) mix_s[e] = a.mix[e];
    pdl_wait();
    const T* qrow = (const T*)a.q + (size_t)b * a.q_stride;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) q_s[e] = to_f<T>(qrow[e]);
    __syncthreads();
    const int len = a.len_after[b];
    const int lo = first_seen(a.window, len - 1);
    int per = (len - lo + a.n_pieces - 1) / a.n_pieces;
    per = (per + 31) & ~31;
    const int beg = lo + piece * per;
    const int end = min(len, beg + per);
    const bool vec = (D % Vec<T>::N) == 0 && (((uintptr_t)a.k) & 15) == 0 && (((uintptr_t)a.v) & 15) == 0;
    const int* pt = a.page_table + (size_t)b * a.pt_stride;
    MixAcc<NC> acc; acc.init();
    int buf = 0;
    for (int j0 = beg; j0 < end; j0 += 32, buf ^= 1) {
        const int j = j0 + lane;
        const bool valid = j < end;
        const T* krow = nullptr; const T* vrow = nullptr;
        if (valid) {
            const int r = a.ring_rows > 0 ? j % a.ring_rows : j;
            const size_t off = (((size_t)pt[r / a.page_rows] * a.G + kvh) * a.page_rows + (r % a.page_rows)) * D;
            krow = (const T*)a.k + off; vrow = (const T*)a.v + off;
        }
        mixed_chunk<T, NC>(acc, q_s + h * D, mix_s + h * H, raw + buf * H * 32, H, h, krow, vrow, valid, D, vec, lane);
    }
    if (a.n_pieces == 1) {
        float inv = 1.f / acc.l;
        if (a.unit_sink) {
            const float M = fmaxf(acc.m, 0.f);
            const float f = expf(acc.m - M);
            inv = f / (acc.l * f + expf(-M));
        }
        T* orow = (T*)a.out + (size_t)b * a.out_stride + (size_t)h * D;
#pragma unroll
        for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < D) orow[d] = from_f<T>(acc.o[c] * inv); }
    } else {
        float* p = a.partial + (((size_t)b * H + h) * a.n_pieces + piece) * (D + 2);
#pragma unroll
        for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < D) p[d] = acc.o[c]; }
        if (lane == 0) { p[D] = acc.m; p[D + 1] = acc.l; }
    }
}

// out[b, h, :] = sum_s e^(m_s - M) o_s / (unit_sink e^(-M) + sum_s e^(m_s - M) l_s), pieces in ascending order.
template <typename T>
__global__ void attn_mixed_fold_kernel(MixedAttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, D = a.D, n = a.n_pieces;
    const float* p = a.partial + ((size_t)b * a.H + h) * n * (D + 2);
    float M = a.unit_sink ? 0.f : -INFINITY;
    for (int s = 0; s < n; s++) M = fmaxf(M, p[(size_t)s * (D + 2) + D]);
    float L = a.unit_sink ? expf(-M) : 0.f;
    for (int s = 0; s < n; s++) {
        const float ms = p[(size_t)s * (D + 2) + D];
        if (ms != -INFINITY) L += p[(size_t)s * (D + 2) + D + 1] * expf(ms - M);
    }
    T* orow = (T*)a.out + (size_t)b * a.out_stride + (size_t)h * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n; s++) {
            const float ms = p[(size_t)s * (D + 2) + D];
            if (ms != -INFINITY) o += p[(size_t)s * (D + 2) + d] * expf(ms - M);
        }
        orow[d] = from_f<T>(o / L);
    }
}

static int pick_nc(int D) {
    const int need = (D + 31) / 32;
    int nc = 1;
    while (nc < need) nc <<= 1;
    return nc;
}

#define MIX_DISPATCH_NC(nc, ...)                                    \
    switch (nc) {                                                   \
    case 1: { constexpr int NC = 1; __VA_ARGS__; } break;           \
    case 2: { constexpr int NC = 2; __VA_ARGS__; } break;           \
    case 4: { constexpr int NC = 4; __VA_ARGS__; } break;           \
    case 8: { constexpr int NC = 8; __VA_ARGS__; } break;           \
    default: { constexpr int NC = 16; __VA_ARGS__; } break;         \
    }

static int check_shape(const MixedAttnArgs& a, size_t* smem) {
    if (a.H <= 0 || a.G <= 0 || a.H % a.G != 0) return tb_refuse("attn_mixed: %d heads cannot share %d kv heads", a.H, a.G);
    if (a.H > 32) return tb_refuse("attn_mixed: %d heads are more than the 32 that one CTA mixes", a.H);
    if (a.D <= 0 || a.D > 512) return tb_refuse("attn_mixed: head size %d is outside [1, 512]", a.D);
    if (a.mix == nullptr) return tb_refuse("attn_mixed: no mixing matrix");
    *smem = ((size_t)a.H * a.D + (size_t)a.H * a.H + 2 * (size_t)a.H * 32) * sizeof(float);
    if (*smem > 200 * 1024) return tb_refuse("attn_mixed: %d heads of %d numbers do not fit a CTA's shared memory", a.H, a.D);
    return 0;
}

template <typename K>
static void allow_smem(K kern, size_t smem) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

extern "C" int tb_attn_mixed_prefill(const MixedAttnArgs* args, int dtype, cudaStream_t stream) {
    const MixedAttnArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    size_t smem = 0;
    if (check_shape(a, &smem)) return -1;
    const int nc = pick_nc(a.D);
    TB_DISPATCH_1(dtype, T, MIX_DISPATCH_NC(nc,
        allow_smem(attn_mixed_prefill_kernel<T, NC>, smem);
        tb_launch(attn_mixed_prefill_kernel<T, NC>, dim3(a.n_tokens), dim3(a.H * 32), smem, stream, a)));
    return tb_launch_status();
}

extern "C" int tb_attn_mixed_decode(const MixedAttnArgs* args, int dtype, cudaStream_t stream) {
    const MixedAttnArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    size_t smem = 0;
    if (check_shape(a, &smem)) return -1;
    if (a.n_pieces < 1 || a.n_pieces > 65535) return tb_refuse("attn_mixed: pieces=%d", a.n_pieces);
    if (a.n_pieces > 1 && a.partial == nullptr) return tb_refuse("attn_mixed: pieces need scratch");
    if (a.page_rows <= 0 || (a.ring_rows > 0 && a.ring_rows % a.page_rows))
        return tb_refuse("attn_mixed: page_rows=%d ring_rows=%d", a.page_rows, a.ring_rows);
    if (a.ring_rows > 0 && (a.window == 0 || abs(a.window) > a.ring_rows))
        return tb_refuse("attn_mixed: a ring of %d rows cannot hold a window of %d", a.ring_rows, abs(a.window));
    const int nc = pick_nc(a.D);
    TB_DISPATCH_1(dtype, T, MIX_DISPATCH_NC(nc,
        allow_smem(attn_mixed_decode_kernel<T, NC>, smem);
        tb_launch(attn_mixed_decode_kernel<T, NC>, dim3(a.n_tokens, a.n_pieces), dim3(a.H * 32), smem, stream, a)));
    int st = tb_launch_status();
    if (st || a.n_pieces == 1) return st;
    TB_DISPATCH_1(dtype, T, tb_launch(attn_mixed_fold_kernel<T>, dim3(a.n_tokens, a.H), dim3(128), 0, stream, a));
    return tb_launch_status();
}
