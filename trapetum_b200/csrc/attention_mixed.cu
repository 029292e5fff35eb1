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
//   tb_attn_mixed_prefill   queries and keys are the step's own packed tokens; in bfloat16 with up to 16 heads of 32, 64,
//                           96 or 128 numbers the dot products run on tensor cores (mma.sync): a CTA takes 16 queries
//                           of all heads, a warp a head; raw scores of 32 keys go through shared memory, every
//                           warp mixes its own head's in 32-bit, keeps the running softmax in registers and multiplies
//                           the rounded weights with the values
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
    int batch, max_seq_len;                               // prefill on tensor cores: sequences of the step, the longest's tokens
    int stages;                                           // ... and how many rounds' keys and values lie in shared memory (set by the library)
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
        float d4[4] = {0.f, 0.f, 0.f, 0.f};              // four sums side by side: no product waits for the one before it
        for (int e = 0; e < D; e += N) {
            const uint4 u = *(const uint4*)(krow + e);
            const T* x = (const T*)&u;
            __align__(16) float qv[N];                   // the query from shared memory 16 bytes at a time (every lane the same)
#pragma unroll
            for (int i = 0; i < N; i += 4) *(float4*)(qv + i) = *(const float4*)(q_s + e + i);
#pragma unroll
            for (int i = 0; i < N; i++) d4[i & 3] = fmaf(qv[i], to_f<T>(x[i]), d4[i & 3]);
        }
        d = (d4[0] + d4[1]) + (d4[2] + d4[3]);
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
    // a lane owns the NC consecutive dims from lane * NC on; with whole 16-byte rows it reads them in one piece
    constexpr int BYTES = NC * (int)sizeof(T);
    const bool wide = vec && (D % NC) == 0 && (BYTES == 4 || BYTES == 8 || BYTES % 16 == 0);
    const int d0 = lane * NC;
    for (int jj = 0; jj < 32; jj++) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)vrow, jj);
        if (pj == 0.f) continue;
        const T* v = (const T*)(uintptr_t)vp;
        if (wide) {
            if (d0 < D) {
                __align__(16) T x[NC];
                if (BYTES == 4) *(uint32_t*)x = *(const uint32_t*)(v + d0);
                else if (BYTES == 8) *(uint2*)x = *(const uint2*)(v + d0);
                else {
#pragma unroll
                    for (int i = 0; i < BYTES / 16; i++) ((uint4*)x)[i] = ((const uint4*)(v + d0))[i];
                }
#pragma unroll
                for (int c = 0; c < NC; c++) acc.o[c] = fmaf(pj, to_f<T>(x[c]), acc.o[c]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = d0 + c;
                if (d < D) acc.o[c] = fmaf(pj, to_f<T>(v[d]), acc.o[c]);
            }
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
        const int d = lane * NC + c;
        if (d < D) orow[d] = from_f<T>(acc.o[c] * inv);
    }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                        // 0: sixteen zero bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n) : "memory");
}

// The keys and values of 32 rows for all kv heads at once: rows of D numbers padded by 16 bytes, [K | V][G][32][pitch].
template <typename T>
__host__ __device__ constexpr int tile_pitch(int D) { return D + 16 / (int)sizeof(T); }

// STAGED: a tile of 32 cached rows of every kv head is copied into shared memory (16 bytes a thread and copy, the
// next tile on its way while this one is used), so that the rows are fetched once for all heads and with whole
// lines; else every lane reads its key's row from the cache itself (any size and alignment).
template <typename T, int NC, bool STAGED>
__global__ void attn_mixed_decode_kernel(MixedAttnArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float smem[];
    const int H = a.H, D = a.D;
    float* q_s = smem;
    float* mix_s = q_s + H * D;
    float* raw = mix_s + H * H;
    T* tiles = (T*)(((uintptr_t)(raw + 2 * H * 32) + 15) & ~(uintptr_t)15);      // [2 stages][K | V][G][32][pitch]
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
    if (STAGED) {
        const int pitch = tile_pitch<T>(D), per_row = D * (int)sizeof(T) / 16;
        const size_t stage = (size_t)2 * a.G * 32 * pitch;
        auto load = [&](int st, int j0) {
            T* dst = tiles + st * stage;
            for (int c = threadIdx.x; c < 2 * a.G * 32 * per_row; c += blockDim.x) {
                const int ch = c % per_row, row = (c / per_row) % 32, g = (c / per_row / 32) % a.G, kv = c / per_row / 32 / a.G;
                const int j = j0 + row;
                const bool ok = j < end;
                const int r = ok ? (a.ring_rows > 0 ? j % a.ring_rows : j) : 0;
                const size_t off = (((size_t)pt[r / a.page_rows] * a.G + g) * a.page_rows + (r % a.page_rows)) * D;
                cp_async16(dst + ((size_t)(kv * a.G + g) * 32 + row) * pitch + ch * (16 / sizeof(T)),
                           (const T*)(kv ? a.v : a.k) + off + ch * (16 / sizeof(T)), ok);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (beg < end) load(0, beg);
        int st = 0;
        for (int j0 = beg; j0 < end; j0 += 32, buf ^= 1, st ^= 1) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();                             // the tile is there, and nobody reads the other stage any more
            if (j0 + 32 < end) load(st ^ 1, j0 + 32);
            const bool valid = j0 + lane < end;
            const T* krow = tiles + st * stage + ((size_t)kvh * 32 + lane) * pitch;
            const T* vrow = krow + (size_t)a.G * 32 * pitch;
            mixed_chunk<T, NC>(acc, q_s + h * D, mix_s + h * H, raw + buf * H * 32, H, h, krow, vrow, valid, D, true, lane);
        }
    } else
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
        for (int c = 0; c < NC; c++) { const int d = lane * NC + c; if (d < D) orow[d] = from_f<T>(acc.o[c] * inv); }
    } else {
        float* p = a.partial + (((size_t)b * H + h) * a.n_pieces + piece) * (D + 2);
#pragma unroll
        for (int c = 0; c < NC; c++) { const int d = lane * NC + c; if (d < D) p[d] = acc.o[c]; }
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


// ---------------------------------------------------------------------------
// Prompts on tensor cores (bfloat16; H <= 32 heads; D = 16 KT).  16 queries a CTA, a warp a head, 32 keys a round.
// With more than 16 heads two CTAs (along z) share a tile of queries: each makes the raw scores of ALL heads (a warp
// those of heads w and w + 16; the second one's queries come from memory every round, not from registers), because
// every head's mixed score needs them all, and mixes, weighs and writes 16 heads of its own.
// ---------------------------------------------------------------------------
constexpr int MP_BM = 16, MP_BN = 32, MP_RP = 40;        // raw scores' row pitch: 8 mod 32 words keeps a warp's 8-byte accesses apart

__device__ __forceinline__ void mp_ldsm2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mp_ldsm4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mp_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t mp_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}

// How many kv heads' values a CTA keeps: all of them with up to 16 heads, else those of 16 consecutive heads.
__host__ __device__ inline int mp_value_heads(int H, int G) {
    if (H <= 16) return G;
    const int per = H / G, n = 15 / per + 2;
    return n < G ? n : G;
}
__host__ inline size_t mp_smem(int H, int G, int D, int stages) {
    return (size_t)((H * H + 3) & ~3) * 4 + (size_t)H * MP_BM * MP_RP * 4 + (size_t)stages * (G + mp_value_heads(H, G)) * MP_BN * (D + 8) * 2;
}

// MULTI: more than 16 heads (the second paragraph above); else a warp's only raw scores are its own head's.
template <int KT, bool MULTI>
__global__ void __launch_bounds__(512) attn_mixed_prefill_mma_kernel(MixedAttnArgs a) {
    pdl_launch_dependents();
    constexpr int D = 16 * KT, PITCH = D + 8;
    extern __shared__ __align__(16) unsigned char sm[];
    const int H = a.H, G = a.G, GV = mp_value_heads(H, G);
    float* mix_s = (float*)sm;                                        // [H][H]
    float* raw = mix_s + ((H * H + 3) & ~3);                          // [H][16][MP_RP]
    bf16* tiles = (bf16*)(raw + H * MP_BM * MP_RP);                   // [stages][K: G | V: GV][32][PITCH]
    const size_t k_part = (size_t)G * MP_BN * PITCH, stage = k_part + (size_t)GV * MP_BN * PITCH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h_raw = warp < H ? warp : 0;
    const int h_out = blockIdx.z * 16 + warp;                         // the head this warp mixes, weighs and writes
    const bool has_out = h_out < H;
    const int h = has_out ? h_out : h_raw;                            // the head whose queries stay in registers
    const int r = lane >> 2, c = (lane & 3) * 2;                      // this thread's rows r and r + 8, columns c and c + 1 of a tile of 8
    const int per_kv = H / G;
    const int kv_lo = (blockIdx.z * 16) / per_kv;                     // the first kv head whose values this CTA needs
    const int kvh = h / per_kv;
    for (int e = threadIdx.x; e < H * H; e += blockDim.x) mix_s[e] = a.mix[e];
    pdl_wait();
    const int b = blockIdx.y;
    const int s0 = a.seq_start[b], len = a.seq_start[b + 1] - s0;
    // a tile's keys may be cut into pieces that CTAs of their own take (a short prompt then fills the GPU); their
    // partial (max, sum, o) are folded by attn_mixed_fold_kernel, in piece order
    const int P = a.n_pieces > 1 ? a.n_pieces : 1;
    const int i0 = (blockIdx.x / P) * MP_BM, piece = blockIdx.x % P;
    if (i0 >= len) return;
    const int i_last = min(i0 + MP_BM - 1, len - 1);
    const int ia = i0 + r, ib = i0 + r + 8;                           // the two queries whose scores this thread holds
    // the queries of this head as the products' left operand, kept in registers
    uint32_t qf[KT][4];
    {
        const bf16* qa = (const bf16*)a.q + (size_t)(s0 + ia) * a.q_stride + (size_t)h * D + c;
        const bf16* qb = (const bf16*)a.q + (size_t)(s0 + ib) * a.q_stride + (size_t)h * D + c;
#pragma unroll
        for (int k = 0; k < KT; k++) {
            qf[k][0] = ia < len ? *(const uint32_t*)(qa + k * 16) : 0u;
            qf[k][1] = ib < len ? *(const uint32_t*)(qb + k * 16) : 0u;
            qf[k][2] = ia < len ? *(const uint32_t*)(qa + k * 16 + 8) : 0u;
            qf[k][3] = ib < len ? *(const uint32_t*)(qb + k * 16 + 8) : 0u;
        }
    }
    float o[2 * KT][4];
#pragma unroll
    for (int n = 0; n < 2 * KT; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;     // l: this thread's share, summed over the four at the end
    const int lo_a = first_seen(a.window, ia), lo_b = first_seen(a.window, ib);
    const float* mix_row = mix_s + h * H;
    constexpr int PER_ROW = D / 8;                                    // 16-byte pieces of a row
    // keys of 32 positions for every kv head and values for this CTA's; with two stages the next round's are on their
    // way while this round computes
    auto load = [&](int st, int j0) {
        bf16* dst = tiles + st * stage;
        for (int p = threadIdx.x; p < (G + GV) * MP_BN * PER_ROW; p += blockDim.x) {
            const int ch = p % PER_ROW, row = (p / PER_ROW) % MP_BN, gg = p / PER_ROW / MP_BN;
            const bool is_v = gg >= G;
            const int g = is_v ? kv_lo + gg - G : gg;
            const bool ok = j0 + row <= i_last && g < G;
            const bf16* src = (const bf16*)(is_v ? a.v : a.k) + (size_t)(s0 + (ok ? j0 + row : 0)) * a.kv_stride + (size_t)(ok ? g : 0) * D + ch * 8;
            cp_async16(dst + ((size_t)gg * MP_BN + row) * PITCH + ch * 8, src, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int j_tile = first_seen(a.window, i0);
    const int per = (((i_last - j_tile) / MP_BN + 1) + P - 1) / P;    // rounds a piece
    const int j_first = j_tile + piece * per * MP_BN;
    const int j_stop = min(i_last, j_first + per * MP_BN - 1);
    const bool two = a.stages >= 2;
    if (two && j_first <= j_stop) load(0, j_first);
    int st = 0;
    for (int j0 = j_first; j0 <= j_stop; j0 += MP_BN, st ^= (two ? 1 : 0)) {
        if (!two) { __syncthreads(); load(0, j0); }                   // one stage: the round before must have read it
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                              // this round's tiles are there; the round before has read its own and the raw scores
        if (two && j0 + MP_BN <= j_stop) load(st ^ 1, j0 + MP_BN);
        const uint32_t t_base = (uint32_t)__cvta_generic_to_shared(tiles + st * stage);
        const uint32_t v_base = t_base + (uint32_t)((k_part + (size_t)(kvh - kv_lo) * MP_BN * PITCH) * 2);
        // ---- raw scores of this head: 16 queries x 32 keys
        float sc[4][4];
        for (int hr = warp; hr < (MULTI ? H : warp + 1); hr += 16) {  // the heads whose raw scores this warp makes
#pragma unroll
            for (int nt = 0; nt < 4; nt++) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
            const uint32_t ka = t_base + (uint32_t)((((size_t)(hr / per_kv) * MP_BN + (lane & 7)) * PITCH + ((lane >> 3) & 1) * 8) * 2);
            const bool mine = !MULTI || hr == h;                       // its queries are in registers; the other head's come from memory
            const bf16* qa = (const bf16*)a.q + (size_t)(s0 + ia) * a.q_stride + (size_t)hr * D + c;
            const bf16* qb = (const bf16*)a.q + (size_t)(s0 + ib) * a.q_stride + (size_t)hr * D + c;
#pragma unroll
            for (int ks = 0; ks < KT; ks++) {                          // the four tiles of 8 keys side by side: four sums in flight
                uint32_t qq[4];
                if (mine) { qq[0] = qf[ks][0]; qq[1] = qf[ks][1]; qq[2] = qf[ks][2]; qq[3] = qf[ks][3]; }
                else {
                    qq[0] = ia < len ? *(const uint32_t*)(qa + ks * 16) : 0u; qq[1] = ib < len ? *(const uint32_t*)(qb + ks * 16) : 0u;
                    qq[2] = ia < len ? *(const uint32_t*)(qa + ks * 16 + 8) : 0u; qq[3] = ib < len ? *(const uint32_t*)(qb + ks * 16 + 8) : 0u;
                }
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    uint32_t b0, b1;
                    mp_ldsm2(ka + (uint32_t)(nt * 8 * PITCH * 2) + ks * 32, b0, b1);
                    mp_mma(sc[nt], qq, b0, b1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                float* ra = raw + ((size_t)hr * MP_BM + r) * MP_RP + nt * 8 + c;
                *(float2*)ra = make_float2(sc[nt][0], sc[nt][1]);
                *(float2*)(ra + 8 * MP_RP) = make_float2(sc[nt][2], sc[nt][3]);
            }
        }
        __syncthreads();
        if (MULTI && !has_out) continue;                               // a warp without a head of its own only made raw scores
        // ---- this head's mixed scores, 32-bit
#pragma unroll
        for (int nt = 0; nt < 4; nt++) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
        for (int g = 0; g < H; g++) {
            const float w = mix_row[g];
            const float* ra = raw + ((size_t)g * MP_BM + r) * MP_RP + c;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const float2 x = *(const float2*)(ra + nt * 8), y = *(const float2*)(ra + nt * 8 + 8 * MP_RP);
                sc[nt][0] = fmaf(w, x.x, sc[nt][0]); sc[nt][1] = fmaf(w, x.y, sc[nt][1]);
                sc[nt][2] = fmaf(w, y.x, sc[nt][2]); sc[nt][3] = fmaf(w, y.y, sc[nt][3]);
            }
        }
        // ---- who sees whom, and the running softmax of the two rows
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int j = j0 + nt * 8 + c + e;
                if (!(j <= ia && j >= lo_a)) sc[nt][e] = -INFINITY;
                if (!(j <= ib && j >= lo_b)) sc[nt][2 + e] = -INFINITY;
                mx_a = fmaxf(mx_a, sc[nt][e]); mx_b = fmaxf(mx_b, sc[nt][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
        const float corr_a = m_a == -INFINITY ? 0.f : expf(m_a - ref_a), corr_b = m_b == -INFINITY ? 0.f : expf(m_b - ref_b);
        m_a = mn_a; m_b = mn_b;
        uint32_t pa[2][4];
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const float p0 = expf(sc[nt][0] - ref_a), p1 = expf(sc[nt][1] - ref_a);      // exp(-inf) = 0 for what is not seen
            const float p2 = expf(sc[nt][2] - ref_b), p3 = expf(sc[nt][3] - ref_b);
            sum_a += p0 + p1; sum_b += p2 + p3;
            pa[nt >> 1][(nt & 1) * 2] = mp_pack(p0, p1);
            pa[nt >> 1][(nt & 1) * 2 + 1] = mp_pack(p2, p3);
        }
        l_a = l_a * corr_a + sum_a; l_b = l_b * corr_b + sum_b;
        // ---- O = O * corr + P V
#pragma unroll
        for (int n = 0; n < 2 * KT; n++) { o[n][0] *= corr_a; o[n][1] *= corr_a; o[n][2] *= corr_b; o[n][3] *= corr_b; }
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {                               // all tiles of the values' dims side by side
#pragma unroll
            for (int dn = 0; dn < KT; dn++) {
                uint32_t b0, b1, b2, b3;
                mp_ldsm4_t(v_base + (uint32_t)(((kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PITCH + dn * 16 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                mp_mma(o[2 * dn], pa[kk], b0, b1);
                mp_mma(o[2 * dn + 1], pa[kk], b2, b3);
            }
        }
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (P > 1) {
        if (MULTI && !has_out) return;
        float* pa_row = a.partial + (((size_t)(s0 + ia) * H + h) * P + piece) * (D + 2);
        float* pb_row = a.partial + (((size_t)(s0 + ib) * H + h) * P + piece) * (D + 2);
#pragma unroll
        for (int n = 0; n < 2 * KT; n++) {
            if (ia < len) *(float2*)(pa_row + n * 8 + c) = make_float2(o[n][0], o[n][1]);
            if (ib < len) *(float2*)(pb_row + n * 8 + c) = make_float2(o[n][2], o[n][3]);
        }
        if ((lane & 3) == 0) {
            if (ia < len) { pa_row[D] = m_a; pa_row[D + 1] = l_a; }
            if (ib < len) { pb_row[D] = m_b; pb_row[D + 1] = l_b; }
        }
        return;
    }
    float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
    if (a.unit_sink) {
        // the denominator also holds exp(0); the sums stand relative to the rows' maxima
        const float Ma = fmaxf(m_a, 0.f), Mb = fmaxf(m_b, 0.f);
        const float fa = expf(m_a - Ma), fb = expf(m_b - Mb);
        inv_a = fa / (l_a * fa + expf(-Ma)); inv_b = fb / (l_b * fb + expf(-Mb));
    }
    if (!has_out) return;
    bf16* oa_row = (bf16*)a.out + (size_t)(s0 + ia) * a.out_stride + (size_t)h * D + c;
    bf16* ob_row = (bf16*)a.out + (size_t)(s0 + ib) * a.out_stride + (size_t)h * D + c;
#pragma unroll
    for (int n = 0; n < 2 * KT; n++) {
        if (ia < len) *(uint32_t*)(oa_row + n * 8) = mp_pack(o[n][0] * inv_a, o[n][1] * inv_a);
        if (ib < len) *(uint32_t*)(ob_row + n * 8) = mp_pack(o[n][2] * inv_b, o[n][3] * inv_b);
    }
}

// Whether the tensor-core form takes a step's shapes (the generic kernel takes the rest).
extern "C" int tb_attn_mixed_prefill_mma_takes(int dtype, int H, int G, int D) {
    if (dtype != TB_BF16 || H < 1 || H > 32 || G < 1 || H % G || D % 32 || D < 32 || D > 128) return 0;
    return mp_smem(H, G, D, 1) <= 200 * 1024;
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
    *smem = (((size_t)a.H * a.D + (size_t)a.H * a.H + 2 * (size_t)a.H * 32) * sizeof(float) + 15) / 16 * 16;
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
    const bool aligned = (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.out) & 15) == 0 && a.q_stride % 8 == 0
        && a.kv_stride % 8 == 0 && a.out_stride % 8 == 0;
    if (a.batch > 0 && a.max_seq_len > 0 && aligned && tb_attn_mixed_prefill_mma_takes(dtype, a.H, a.G, a.D)) {
        MixedAttnArgs am = a;
        am.stages = mp_smem(a.H, a.G, a.D, 2) <= 200 * 1024 ? 2 : 1;
        const size_t sm = mp_smem(a.H, a.G, a.D, am.stages);
        if (am.n_pieces > 1 && a.partial == nullptr) return tb_refuse("attn_mixed: pieces need scratch");
        if (am.n_pieces < 1) am.n_pieces = 1;
        dim3 grid((a.max_seq_len + MP_BM - 1) / MP_BM * am.n_pieces, a.batch, (a.H + 15) / 16);
        const int warps = a.H < 16 ? a.H : 16;
#define TB_MP_LAUNCH(KT) do { if (a.H > 16) { allow_smem(attn_mixed_prefill_mma_kernel<KT, true>, sm); \
            tb_launch(attn_mixed_prefill_mma_kernel<KT, true>, grid, dim3(warps * 32), sm, stream, am); } \
        else { allow_smem(attn_mixed_prefill_mma_kernel<KT, false>, sm); \
            tb_launch(attn_mixed_prefill_mma_kernel<KT, false>, grid, dim3(warps * 32), sm, stream, am); } } while (0)
        switch (a.D / 16) { case 2: TB_MP_LAUNCH(2); break; case 4: TB_MP_LAUNCH(4); break; case 6: TB_MP_LAUNCH(6); break; default: TB_MP_LAUNCH(8); break; }
#undef TB_MP_LAUNCH
        int st = tb_launch_status();
        if (st || am.n_pieces == 1) return st;
        TB_DISPATCH_1(dtype, T, tb_launch(attn_mixed_fold_kernel<T>, dim3(a.n_tokens, a.H), dim3(128), 0, stream, am));
        return tb_launch_status();
    }
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
    // the staged form: rows of whole 16-byte pieces, two stages of every kv head's keys and values within a CTA's memory
    const size_t el = dtype == TB_BF16 ? 2 : 4;
    const size_t tiles = (size_t)2 * 2 * a.G * 32 * (a.D + 16 / el) * el;
    const bool staged = (a.D * el) % 16 == 0 && (((uintptr_t)a.k | (uintptr_t)a.v) & 15) == 0 && smem + tiles <= 160 * 1024;
    if (staged) {
        smem += tiles;
        TB_DISPATCH_1(dtype, T, MIX_DISPATCH_NC(nc,
            allow_smem(attn_mixed_decode_kernel<T, NC, true>, smem);
            tb_launch(attn_mixed_decode_kernel<T, NC, true>, dim3(a.n_tokens, a.n_pieces), dim3(a.H * 32), smem, stream, a)));
    } else
    TB_DISPATCH_1(dtype, T, MIX_DISPATCH_NC(nc,
        allow_smem(attn_mixed_decode_kernel<T, NC, false>, smem);
        tb_launch(attn_mixed_decode_kernel<T, NC, false>, dim3(a.n_tokens, a.n_pieces), dim3(a.H * 32), smem, stream, a)));
    int st = tb_launch_status();
    if (st || a.n_pieces == 1) return st;
    TB_DISPATCH_1(dtype, T, tb_launch(attn_mixed_fold_kernel<T>, dim3(a.n_tokens, a.H), dim3(128), 0, stream, a));
    return tb_launch_status();
}
