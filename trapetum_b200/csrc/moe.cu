// A feed-forward made of experts behind a router.
//
//   tb_moe_route     per token, from the logits z = R x (32-bit sums of a product, given as split-K partial sums):
//                    scores s = sigmoid(z), or softmax(z) over all experts; choice scores s + correction;
//                    experts form `groups` equal groups of neighbours, a group's score is the sum of its
//                    `group_top` largest choice scores, experts outside the `keep` best groups cannot be chosen
//                    (their choice scores count as minus infinity); the `top` largest choice scores win (the
//                    lower index on a tie); weights are the winners' s divided by their sum + eps, times out_scale.  Also the
//                    shared expert's gate sigmoid(g . x), one number per token, if asked for.
//   tb_moe_gate_up   for every (token, chosen expert): silu(G_e x) * (U_e x), or, for experts without a gate matrix,
//                    relu(U_e x)^2
//   tb_moe_down      out[t] = sum_k weight[t,k] * D_e(t,k) a[t,k]  (+ gate[t] * shared[t], the shared expert's output
//                    given as 32-bit split-K partial sums), 32-bit
//
// The router is 32-bit throughout.  The experts' products take operands of the activations' dtype and sum in
// 32-bit; a[t,k] is rounded to the activations' dtype, the weighted sum over the experts is not.
#include "common.cuh"

TB_EXPORT_ERROR()

struct MoeRouteArgs {
    const float* logits; int splits; long long split_stride, row_stride;   // [splits][T][>= E (+ 1)]: 32-bit partial sums of R x
    const float* correction;                   // [E] or null
    int has_gate;                              // column E of the logits is the shared expert's gate g . x
    int* idx; float* weight;                   // [T][top]
    float* gate;                               // [T] (if shared_gate)
    int n_tokens, W, E, top, groups, keep, group_top;
    float weight_eps;
    int softmax;                               // scores are softmax(z) over the experts instead of sigmoid(z)
    float out_scale;                           // the weights times this
    const float* bias;                         // [E] added to the logits themselves, or null
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

__global__ void __launch_bounds__(128) moe_route_kernel(MoeRouteArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    float* score = smem + (size_t)warp * (2 * a.E + a.groups);
    float* choice = score + a.E;
    float* gscore = choice + a.E;
    pdl_wait();
    if (t >= a.n_tokens) return;
    for (int e = lane; e < a.E + (a.has_gate ? 1 : 0); e += 32) {
        const float* src = a.logits + (size_t)t * a.row_stride + e;
        float d = 0.f;
        int sp = 0;
        for (; sp + 4 <= a.splits; sp += 4) {          // four loads on their way at a time, added in split order
            const float v0 = src[(size_t)sp * a.split_stride], v1 = src[(size_t)(sp + 1) * a.split_stride];
            const float v2 = src[(size_t)(sp + 2) * a.split_stride], v3 = src[(size_t)(sp + 3) * a.split_stride];
            d = (((d + v0) + v1) + v2) + v3;
        }
        for (; sp < a.splits; sp++) d += src[(size_t)sp * a.split_stride];
        if (a.bias != nullptr && e < a.E) d += a.bias[e];
        const float s = 1.f / (1.f + expf(-d));
        if (e < a.E) { score[e] = a.softmax ? d : s; choice[e] = s + (a.correction ? a.correction[e] : 0.f); }
        else a.gate[t] = s;
    }
    __syncwarp();
    if (a.softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, score[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < a.E; e += 32) { const float x = expf(score[e] - mx); score[e] = x; sum += x; }
        sum = warp_sum(sum);
        for (int e = lane; e < a.E; e += 32) {
            const float s = score[e] / sum;
            score[e] = s; choice[e] = s + (a.correction ? a.correction[e] : 0.f);
        }
        __syncwarp();
    }
    if (a.groups > 1) {
        const int per = a.E / a.groups;
        for (int g = lane; g < a.groups; g += 32) {
            int used[8];
            float sum = 0.f;
            for (int n = 0; n < a.group_top && n < per; n++) {
                float best = -INFINITY; int bi = -1;
                for (int j = 0; j < per; j++) {
                    bool taken = false;
                    for (int u = 0; u < n; u++) taken |= (used[u] == j);
                    if (!taken && (bi < 0 || choice[g * per + j] > best)) { best = choice[g * per + j]; bi = j; }
                }
                used[n] = bi; sum += best;
            }
            gscore[g] = sum;
        }
        __syncwarp();
        // the `keep` best groups stay; the others' experts cannot be chosen
        unsigned kept_lo = 0;                    // this lane's groups lane, lane+32, ... as bits
        for (int n = 0; n < a.keep; n++) {
            float v = -INFINITY; int i = 0x7fffffff;
            for (int g = lane; g < a.groups; g += 32)
                if (!((kept_lo >> (g >> 5)) & 1u) && (gscore[g] > v || i == 0x7fffffff)) { v = gscore[g]; i = g; }
            warp_argmax(v, i);
            if ((i & 31) == lane && i != 0x7fffffff) kept_lo |= 1u << (i >> 5);
        }
        for (int g = lane; g < a.groups; g += 32)
            if (!((kept_lo >> (g >> 5)) & 1u))
                for (int j = 0; j < per; j++) choice[g * per + j] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f, mine = 0.f; int mine_i = 0;
    for (int n = 0; n < a.top; n++) {
        float v = -INFINITY; int i = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32) if (choice[e] > v) { v = choice[e]; i = e; }
        warp_argmax(v, i);
        const float s = score[i];
        wsum += s;
        if (lane == (n & 31)) { mine = s; mine_i = i; if (n >= 32) { /* more than 32 winners: written below per round */ } }
        __syncwarp();
        if (lane == 0) choice[i] = -INFINITY;
        __syncwarp();
        if ((n & 31) == 31 || n == a.top - 1) {
            // park the round's winners; the weights are divided once the sum is known
            if (lane <= (n & 31)) { a.idx[(size_t)t * a.top + (n & ~31) + lane] = mine_i; a.weight[(size_t)t * a.top + (n & ~31) + lane] = mine; }
        }
    }
    __syncwarp();
    const float inv = a.out_scale / (wsum + a.weight_eps);
    for (int n = lane; n < a.top; n += 32) a.weight[(size_t)t * a.top + n] *= inv;
}

struct MoeExpertArgs {
    const void* x; long long x_stride;         // [T][W]
    const void* gate_w; const void* up_w;      // [E][ff][W]
    const void* down_w;                        // [E][W][ff]
    const int* idx; const float* weight;       // [T][top]
    void* act;                                 // [T * top][ff]
    const float* shared; int shared_splits; long long shared_split_stride;   // [splits][T][W] or null
    const float* gate;                         // [T] (with shared)
    float* out;                                // [T][W]
    int n_tokens, W, ff, top;
    int ungated;                               // experts are D relu(U x)^2: there is no gate matrix
};

// n numbers of the activations' dtype into shared memory as 32-bit, times `scale`, by all threads of the block: 16 bytes
// a load where the dtype is 16-bit, n a multiple of 8 and the source 16-byte aligned.
template <typename T>
__device__ __forceinline__ void fill_f32(float* __restrict__ dst, const T* __restrict__ src, int n, float scale) {
    if (sizeof(T) == 2 && (n & 7) == 0 && (((uintptr_t)src) & 15) == 0) {
        for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
            const uint4 v = *(const uint4*)(src + i);
            const T* e = (const T*)&v;
            *(float4*)(dst + i) = make_float4(to_f<T>(e[0]) * scale, to_f<T>(e[1]) * scale, to_f<T>(e[2]) * scale, to_f<T>(e[3]) * scale);
            *(float4*)(dst + i + 4) = make_float4(to_f<T>(e[4]) * scale, to_f<T>(e[5]) * scale, to_f<T>(e[6]) * scale, to_f<T>(e[7]) * scale);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = to_f<T>(src[i]) * scale;
    }
}

// 16 bytes of a weight row per lane and load where the row allows it; MV_ROWS rows (and for gate/up both matrices) are on
// their way together, so that a warp keeps enough bytes in flight to stream an expert's matrices at the memory's speed.
constexpr int MV_ROWS = 4;

template <typename T>
__device__ __forceinline__ void mv_dot(const T* __restrict__ w0, long long ld, int n_rows, const float* __restrict__ x_s, int K, int lane,
                                       float* acc /* [MV_ROWS] */) {
    constexpr int VEC = 16 / sizeof(T);
#pragma unroll
    for (int r = 0; r < MV_ROWS; r++) acc[r] = 0.f;
    if ((K % VEC) == 0 && ((((uintptr_t)w0) | ((uintptr_t)(ld * sizeof(T))) | (uintptr_t)__cvta_generic_to_shared(x_s)) & 15) == 0) {
        // two steps of the row at once: 2 x MV_ROWS loads of 16 bytes are asked for before the first is used
        for (int c = lane * VEC; c < K; c += 64 * VEC) {
            const int c2 = c + 32 * VEC;
            const bool second = c2 < K;
            uint4 wv[MV_ROWS], wv2[MV_ROWS];
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) wv[r] = r < n_rows ? __ldg((const uint4*)(w0 + (size_t)r * ld + c)) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) wv2[r] = (second && r < n_rows) ? __ldg((const uint4*)(w0 + (size_t)r * ld + c2)) : make_uint4(0, 0, 0, 0);
            // the vector's numbers by 16-byte reads (x_s is 16-byte aligned and K a multiple of VEC): read one by one,
            // a warp's lanes, VEC numbers apart, meet the same bank VEC times
            float xv[VEC];
#pragma unroll
            for (int k = 0; k < VEC; k += 4) {
                const float4 q = *(const float4*)(x_s + c + k);
                xv[k] = q.x; xv[k + 1] = q.y; xv[k + 2] = q.z; xv[k + 3] = q.w;
            }
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) {
                const T* e = (const T*)&wv[r];
#pragma unroll
                for (int k = 0; k < VEC; k++) acc[r] = fmaf(to_f<T>(e[k]), xv[k], acc[r]);
            }
            if (second) {
#pragma unroll
                for (int k = 0; k < VEC; k += 4) {
                    const float4 q = *(const float4*)(x_s + c2 + k);
                    xv[k] = q.x; xv[k + 1] = q.y; xv[k + 2] = q.z; xv[k + 3] = q.w;
                }
#pragma unroll
                for (int r = 0; r < MV_ROWS; r++) {
                    const T* e = (const T*)&wv2[r];
#pragma unroll
                    for (int k = 0; k < VEC; k++) acc[r] = fmaf(to_f<T>(e[k]), xv[k], acc[r]);
                }
            }
        }
    } else {
        for (int c = lane; c < K; c += 32)
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) if (r < n_rows) acc[r] = fmaf(to_f<T>(w0[(size_t)r * ld + c]), x_s[c], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < MV_ROWS; r++) acc[r] = warp_sum(acc[r]);
}

template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(MoeExpertArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float x_s[];              // [W]
    const int pair = blockIdx.x, t = pair / a.top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    pdl_wait();
    const int e = a.idx[pair];
    const T* x = (const T*)a.x + (size_t)t * a.x_stride;
    fill_f32<T>(x_s, x, a.W, 1.f);
    __syncthreads();
    const T* gw = (const T*)a.gate_w + (size_t)e * a.ff * a.W;
    const T* uw = (const T*)a.up_w + (size_t)e * a.ff * a.W;
    for (int f0 = (blockIdx.y * nwarp + warp) * MV_ROWS; f0 < a.ff; f0 += gridDim.y * nwarp * MV_ROWS) {
        const int nr = min(MV_ROWS, a.ff - f0);
        float g[MV_ROWS], u[MV_ROWS];
        if (!a.ungated) mv_dot<T>(gw + (size_t)f0 * a.W, a.W, nr, x_s, a.W, lane, g);
        mv_dot<T>(uw + (size_t)f0 * a.W, a.W, nr, x_s, a.W, lane, u);
        if (lane < nr) {
            float gv = a.ungated ? 0.f : g[0], uv = u[0];
#pragma unroll
            for (int r = 1; r < MV_ROWS; r++) if (lane == r) { gv = a.ungated ? 0.f : g[r]; uv = u[r]; }
            const float y = a.ungated ? fmaxf(uv, 0.f) * fmaxf(uv, 0.f) : gv / (1.f + expf(-gv)) * uv;
            ((T*)a.act)[(size_t)pair * a.ff + f0 + lane] = from_f<T>(y);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(MoeExpertArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float a_s[];              // [top][ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    pdl_wait();
    for (int k = 0; k < a.top; k++)
        fill_f32<T>(a_s + (size_t)k * a.ff, (const T*)a.act + ((size_t)t * a.top + k) * a.ff, a.ff, a.weight[(size_t)t * a.top + k]);
    __syncthreads();
    for (int c0 = (blockIdx.y * nwarp + warp) * MV_ROWS; c0 < a.W; c0 += gridDim.y * nwarp * MV_ROWS) {
        const int nr = min(MV_ROWS, a.W - c0);
        float acc[MV_ROWS] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < a.top; k++) {
            float part[MV_ROWS];
            mv_dot<T>((const T*)a.down_w + ((size_t)a.idx[(size_t)t * a.top + k] * a.W + c0) * a.ff, a.ff, nr, a_s + (size_t)k * a.ff, a.ff, lane, part);
#pragma unroll
            for (int r = 0; r < MV_ROWS; r++) acc[r] += part[r];
        }
        if (lane < nr) {
            float v = acc[0];
#pragma unroll
            for (int r = 1; r < MV_ROWS; r++) if (lane == r) v = acc[r];
            const int c = c0 + lane;
            if (a.shared != nullptr) {
                float sh = 0.f;
                for (int s = 0; s < a.shared_splits; s++) sh += a.shared[(size_t)s * a.shared_split_stride + (size_t)t * a.W + c];
                v = fmaf(a.gate[t], sh, v);
            }
            a.out[(size_t)t * a.W + c] = v;
        }
    }
}

// ---------------------------------------------------------------------------
// Many tokens (bfloat16): the (token, expert) pairs are grouped by expert on the device and every expert's
// pairs go through tensor-core products in tiles of 128 pairs, so that an expert's matrices are read once
// per tile of pairs and not once per pair.  Nothing here depends on values the host knows: the grid is
// sized for the most tiles there can be and the surplus CTAs leave at once.
//
//   tb_moe_group     counts, offsets and the pair list ordered by expert; the table of tiles
//   tb_moe_grouped   act = silu(G_e x) * (U_e x) per pair (one launch), pair outputs D_e act times the pair's
//                    weight in 32-bit (one launch), and their sum per token with the shared expert (one launch)
// ---------------------------------------------------------------------------
constexpr int MG_BM = 128, MG_BN = 128, MG_BK = 64, MG_PITCH = MG_BK * 2 + 16, MG_STAGES = 3, MG_THREADS = 256;
constexpr int MG_STAGE_BYTES = (MG_BM + MG_BN) * MG_PITCH;

struct MoeGroupArgs {
    const int* idx;            // [P] expert of every pair (P = tokens * top)
    int* perm;                 // [P] pairs ordered by expert
    int* tile_expert;          // [max_tiles]
    int* tile_row0;            // [max_tiles] first position in perm
    int* tile_rows;            // [max_tiles] pairs in the tile
    int* n_tiles;              // [1]
    int P, E, max_tiles;
};

__global__ void __launch_bounds__(1024) moe_group_kernel(MoeGroupArgs a) {
    pdl_launch_dependents();
    extern __shared__ int sm[];                       // [E] counts, [E] offsets, [E] cursors, [E] first tile
    int* cnt = sm; int* off = sm + a.E; int* cur = sm + 2 * a.E; int* tile0 = sm + 3 * a.E;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    pdl_wait();
    for (int p = threadIdx.x; p < a.P; p += blockDim.x) atomicAdd(&cnt[a.idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int e = 0; e < a.E; e++) { off[e] = o; tile0[e] = t; o += cnt[e]; t += (cnt[e] + MG_BM - 1) / MG_BM; }
        *a.n_tiles = t;
    }
    __syncthreads();
    // within an expert the pairs keep no particular order: every pair's result depends on its own row only
    for (int p = threadIdx.x; p < a.P; p += blockDim.x) {
        const int e = a.idx[p];
        a.perm[off[e] + atomicAdd(&cur[e], 1)] = p;
    }
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
        const int nt = (cnt[e] + MG_BM - 1) / MG_BM;
        for (int i = 0; i < nt; i++) {
            const int t = tile0[e] + i;
            if (t < a.max_tiles) {
                a.tile_expert[t] = e; a.tile_row0[t] = off[e] + i * MG_BM;
                a.tile_rows[t] = min(MG_BM, cnt[e] - i * MG_BM);
            }
        }
    }
}

__device__ __forceinline__ uint32_t mg_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mg_cp16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                     // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(mg_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void mg_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mg_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct MoeGroupedArgs {
    const bf16* x; long long x_stride;                // [T][W]
    const bf16* gate_w; const bf16* up_w;             // [E][ff][W]
    const bf16* down_w;                               // [E][W][ff]
    const int* perm; const int* tile_expert; const int* tile_row0; const int* tile_rows; const int* n_tiles;
    const float* weight;                              // [P]
    bf16* act;                                        // [P][ff]
    float* pair_out;                                  // [P][W]
    int W, ff, top;
};

// MODE 1: rows of x (by pair / top) times [G_e ; U_e] for 64 columns of ff, then silu(g) * u  ->  act[pair]
// MODE 2: rows of x (by pair / top) times U_e for 128 columns of ff, then relu(u)^2            ->  act[pair]
// MODE 0: rows of act (by pair) times D_e for 128 columns of W, times the pair's weight        ->  pair_out[pair]
// A tile is 128 pairs x 128 weight rows, eight warps (4 x 2) of 32 x 64 each, k in blocks of 64 through a three-stage
// cp.async ring.  GATED lays the weight rows out so that a warp holds a gate column and its up column in one thread:
// rows 64w .. 64w+31 of the tile are gate rows n0 + 32w .., rows 64w+32 .. 64w+63 the up rows of the same columns.
template <int MODE>
__global__ void __launch_bounds__(MG_THREADS, 2) moe_grouped_kernel(MoeGroupedArgs a) {
    constexpr bool GATED = MODE == 1, FROM_X = MODE != 0;
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char mg_ring[];
    __shared__ int row_src[MG_BM];
    const int tile = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp >> 1, wn = warp & 1;
    pdl_wait();
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_expert[tile], row0 = a.tile_row0[tile], rows = a.tile_rows[tile];
    const int K = FROM_X ? a.W : a.ff;
    const int N = FROM_X ? a.ff : a.W;
    const int n0 = blockIdx.y * (GATED ? MG_BN / 2 : MG_BN);
    if (threadIdx.x < MG_BM) row_src[threadIdx.x] = threadIdx.x < rows ? a.perm[row0 + threadIdx.x] : -1;
    __syncthreads();
    const bf16* A = FROM_X ? a.x : a.act;
    const long long a_stride = FROM_X ? a.x_stride : a.ff;
    const bf16* B1 = a.up_w + (size_t)e * a.ff * a.W;
    const bf16* B0 = MODE == 1 ? a.gate_w + (size_t)e * a.ff * a.W : (MODE == 2 ? B1 : a.down_w + (size_t)e * a.W * a.ff);
    auto load = [&](int s, int k0) {
        unsigned char* sa = mg_ring + (size_t)s * MG_STAGE_BYTES; unsigned char* sb = sa + MG_BM * MG_PITCH;
        for (int c = threadIdx.x; c < MG_BM * (MG_BK / 8); c += MG_THREADS) {
            const int r = c >> 3, ch = c & 7, k = k0 + ch * 8;
            const int p = row_src[r];
            const bool ok = p >= 0 && k < K;
            const bf16* src = A + (size_t)(ok ? (FROM_X ? p / a.top : p) : 0) * a_stride + (ok ? k : 0);
            mg_cp16(sa + r * MG_PITCH + ch * 16, src, ok);
        }
        for (int c = threadIdx.x; c < MG_BN * (MG_BK / 8); c += MG_THREADS) {
            const int r = c >> 3, ch = c & 7, k = k0 + ch * 8;
            int n; const bf16* base;
            if (GATED) { n = n0 + (r >> 6) * 32 + (r & 31); base = (r & 32) ? B1 : B0; } else { n = n0 + r; base = B0; }
            const bool ok = n < N && k < K;
            mg_cp16(sb + r * MG_PITCH + ch * 16, base + (size_t)(ok ? n : 0) * K + (ok ? k : 0), ok);
        }
    };
    float acc[2][8][4];
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
        for (int n = 0; n < 8; n++) { acc[m][n][0] = acc[m][n][1] = acc[m][n][2] = acc[m][n][3] = 0.f; }
    const int nk = (K + MG_BK - 1) / MG_BK;
#pragma unroll
    for (int s = 0; s < MG_STAGES - 1; s++) {
        if (s < nk) load(s, s * MG_BK);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kb = 0; kb < nk; kb++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MG_STAGES - 2) : "memory");
        __syncthreads();                               // block kb has landed; everybody is done with block kb - 1
        if (kb + MG_STAGES - 1 < nk) load((kb + MG_STAGES - 1) % MG_STAGES, (kb + MG_STAGES - 1) * MG_BK);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const unsigned char* sa = mg_ring + (size_t)(kb % MG_STAGES) * MG_STAGE_BYTES; const unsigned char* sb = sa + MG_BM * MG_PITCH;
#pragma unroll
        for (int ks = 0; ks < MG_BK / 16; ks++) {
            uint32_t fa[2][4];
#pragma unroll
            for (int m = 0; m < 2; m++)
                mg_ldsm(mg_smem(sa + (wm * 32 + m * 16 + (lane & 15)) * MG_PITCH + (ks * 16 + (lane >> 4) * 8) * 2),
                        fa[m][0], fa[m][1], fa[m][2], fa[m][3]);
#pragma unroll
            for (int n = 0; n < 8; n += 2) {
                uint32_t b0, b1, b2, b3;
                mg_ldsm(mg_smem(sb + (wn * 64 + n * 8 + (lane >> 4) * 8 + (lane & 7)) * MG_PITCH + (ks * 16 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
#pragma unroll
                for (int m = 0; m < 2; m++) { mg_mma(acc[m][n], fa[m], b0, b1); mg_mma(acc[m][n + 1], fa[m], b2, b3); }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int cq = (lane & 3) * 2;
#pragma unroll
    for (int m = 0; m < 2; m++) {
        const int ra = wm * 32 + m * 16 + (lane >> 2), rb = ra + 8;
        const int pa = row_src[ra], pb = row_src[rb];
        if (GATED) {
#pragma unroll
            for (int n = 0; n < 4; n++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int col = n0 + wn * 32 + n * 8 + cq + j;
                    if (col >= N) continue;
                    const float ga = acc[m][n][j], ua = acc[m][n + 4][j], gb = acc[m][n][2 + j], ub = acc[m][n + 4][2 + j];
                    if (pa >= 0) a.act[(size_t)pa * a.ff + col] = __float2bfloat16_rn(ga / (1.f + expf(-ga)) * ua);
                    if (pb >= 0) a.act[(size_t)pb * a.ff + col] = __float2bfloat16_rn(gb / (1.f + expf(-gb)) * ub);
                }
            }
        } else if (MODE == 2) {
#pragma unroll
            for (int n = 0; n < 8; n++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int col = n0 + wn * 64 + n * 8 + cq + j;
                    if (col >= N) continue;
                    const float ua = fmaxf(acc[m][n][j], 0.f), ub = fmaxf(acc[m][n][2 + j], 0.f);
                    if (pa >= 0) a.act[(size_t)pa * a.ff + col] = __float2bfloat16_rn(ua * ua);
                    if (pb >= 0) a.act[(size_t)pb * a.ff + col] = __float2bfloat16_rn(ub * ub);
                }
            }
        } else {
            const float wa = pa >= 0 ? a.weight[pa] : 0.f, wb = pb >= 0 ? a.weight[pb] : 0.f;
#pragma unroll
            for (int n = 0; n < 8; n++) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int col = n0 + wn * 64 + n * 8 + cq + j;
                    if (col >= N) continue;
                    if (pa >= 0) a.pair_out[(size_t)pa * a.W + col] = acc[m][n][j] * wa;
                    if (pb >= 0) a.pair_out[(size_t)pb * a.W + col] = acc[m][n][2 + j] * wb;
                }
            }
        }
    }
}

__global__ void moe_sum_pairs_kernel(const float* __restrict__ pair_out, const float* __restrict__ shared, int shared_splits,
                                     long long shared_split_stride, const float* __restrict__ gate, float* __restrict__ out,
                                     long long n, int W, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / W; const int c = (int)(i % W);
    float acc = 0.f;
    for (int k = 0; k < top; k++) acc += pair_out[((size_t)t * top + k) * W + c];      // in the order of the choice
    if (shared != nullptr) {
        float sh = 0.f;
        for (int s = 0; s < shared_splits; s++) sh += shared[(size_t)s * shared_split_stride + i];
        acc = fmaf(gate[t], sh, acc);
    }
    out[i] = acc;
}

// ---------------------------------------------------------------------------
// The same grouping for the tcgen05 product (gemm_tc.cu, grouped mode): the pairs are laid out expert by expert
// with every expert's stretch padded to whole tiles of 128 rows, so that a tile of the product's token operand
// belongs to one expert.  tb_moe_group_padded makes the layout (where every pair goes, which pair every row
// holds, every tile's expert), tb_moe_gather_rows fills the operand, and tb_moe_combine_sorted adds a token's
// weighted expert outputs (and the shared expert) back up.
// ---------------------------------------------------------------------------
struct MoePadArgs {
    const int* idx;            // [P] expert of every pair
    int* pos;                  // [P] the pair's row in the padded order
    int* row_pair;             // [max_rows] the pair a row holds, -1 for padding
    int* tile_group;           // [max_rows / 128] the tile's expert (-1 for tiles past the last one: the product leaves them out)
    int P, E, max_rows;
};

__global__ void __launch_bounds__(1024) moe_group_padded_kernel(MoePadArgs a) {
    pdl_launch_dependents();
    extern __shared__ int sm[];                       // [E] counts, [E] first rows, [E] cursors
    int* cnt = sm; int* off = sm + a.E; int* cur = sm + 2 * a.E;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    pdl_wait();
    for (int r = threadIdx.x; r < a.max_rows; r += blockDim.x) a.row_pair[r] = -1;
    for (int t = threadIdx.x; t < a.max_rows / 128; t += blockDim.x) a.tile_group[t] = -1;     // not in use until an expert claims it
    for (int p = threadIdx.x; p < a.P; p += blockDim.x) atomicAdd(&cnt[a.idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < a.E; e++) { off[e] = o; o += (cnt[e] + 127) / 128 * 128; }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < a.P; p += blockDim.x) {
        const int e = a.idx[p];
        const int r = off[e] + atomicAdd(&cur[e], 1);
        a.pos[p] = r; a.row_pair[r] = p;
    }
    for (int e = threadIdx.x; e < a.E; e += blockDim.x)
        for (int t = off[e] / 128; t < (off[e] + cnt[e] + 127) / 128; t++) a.tile_group[t] = e;
}

__global__ void __launch_bounds__(128) moe_gather_rows_kernel(const bf16* __restrict__ x, long long x_stride, const int* __restrict__ row_pair,
                                                              bf16* __restrict__ out, int W, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int p = row_pair[r];
    uint4* dst = (uint4*)(out + (size_t)r * W);
    if (p < 0) { for (int c = threadIdx.x; c < W / 8; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0); return; }
    const uint4* src = (const uint4*)(x + (size_t)(p / top) * x_stride);
    for (int c = threadIdx.x; c < W / 8; c += blockDim.x) dst[c] = src[c];
}

__global__ void moe_combine_sorted_kernel(const float* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ weight,
                                          const float* __restrict__ shared, int shared_splits, long long shared_split_stride,
                                          const float* __restrict__ gate, float* __restrict__ out, long long n, int W, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / W; const int c = (int)(i % W);
    float acc = 0.f;
    for (int k = 0; k < top; k++) acc = fmaf(weight[t * top + k], y[(size_t)pos[t * top + k] * W + c], acc);   // in the order of the choice
    if (shared != nullptr) {
        float sh = 0.f;
        for (int s = 0; s < shared_splits; s++) sh += shared[(size_t)s * shared_split_stride + i];
        acc = fmaf(gate[t], sh, acc);
    }
    out[i] = acc;
}

extern "C" int tb_moe_group_padded(const MoePadArgs* args, cudaStream_t stream) {
    const MoePadArgs& a = *args;
    if (a.P <= 0) return 0;
    if (a.E <= 0 || a.E > 2048 || a.max_rows % 128 || a.max_rows < a.P) return tb_refuse("moe_group_padded: experts=%d rows=%d", a.E, a.max_rows);
    tb_launch(moe_group_padded_kernel, dim3(1), dim3(1024), (size_t)3 * a.E * sizeof(int), stream, a);
    return tb_launch_status();
}

extern "C" int tb_moe_gather_rows(const void* x, long long x_stride, const int* row_pair, void* out, int rows, int W, int top,
                                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (W % 8 || x_stride % 8 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return tb_refuse("moe_gather_rows: rows must be 16-byte aligned");
    tb_launch(moe_gather_rows_kernel, dim3(rows), dim3(128), 0, stream, (const bf16*)x, x_stride, row_pair, (bf16*)out, W, top);
    return tb_launch_status();
}

extern "C" int tb_moe_combine_sorted(const float* y, const int* pos, const float* weight, const float* shared, int shared_splits,
                                     long long shared_split_stride, const float* gate, float* out, int n_tokens, int W, int top,
                                     cudaStream_t stream) {
    const long long n = (long long)n_tokens * W;
    if (n <= 0) return 0;
    tb_launch(moe_combine_sorted_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, y, pos, weight, shared, shared_splits,
              shared_split_stride, gate, out, n, W, top);
    return tb_launch_status();
}

extern "C" int tb_moe_group(const MoeGroupArgs* args, cudaStream_t stream) {
    const MoeGroupArgs& a = *args;
    if (a.P <= 0) return 0;
    if (a.E <= 0 || a.E > 2048) return tb_refuse("moe_group: %d experts", a.E);
    tb_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)4 * a.E * sizeof(int), stream, a);
    return tb_launch_status();
}

extern "C" int tb_moe_grouped(const MoeGroupedArgs* args, const float* shared, int shared_splits, long long shared_split_stride,
                              const float* gate, float* out, int n_tokens, int max_tiles, cudaStream_t stream) {
    const MoeGroupedArgs& a = *args;
    if (n_tokens <= 0) return 0;
    if (a.W % 8 || a.ff % 8 || ((uintptr_t)a.x & 15) || (a.x_stride % 8))
        return tb_refuse("moe_grouped: W=%d and ff=%d must be multiples of 8 and the rows 16-byte aligned", a.W, a.ff);
    constexpr int SMEM = MG_STAGES * MG_STAGE_BYTES;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e1 = cudaFuncSetAttribute(moe_grouped_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        cudaError_t e2 = cudaFuncSetAttribute(moe_grouped_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        cudaError_t e3 = cudaFuncSetAttribute(moe_grouped_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) return (int)(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3));
        attr_set = true;
    }
    if (a.gate_w != nullptr) tb_launch(moe_grouped_kernel<1>, dim3(max_tiles, (a.ff + 63) / 64), dim3(MG_THREADS), SMEM, stream, a);
    else tb_launch(moe_grouped_kernel<2>, dim3(max_tiles, (a.ff + MG_BN - 1) / MG_BN), dim3(MG_THREADS), SMEM, stream, a);   // experts without a gate matrix
    int st = tb_launch_status();
    if (st) return st;
    tb_launch(moe_grouped_kernel<0>, dim3(max_tiles, (a.W + MG_BN - 1) / MG_BN), dim3(MG_THREADS), SMEM, stream, a);
    st = tb_launch_status();
    if (st) return st;
    const long long n = (long long)n_tokens * a.W;
    tb_launch(moe_sum_pairs_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)a.pair_out, shared,
              shared_splits, shared_split_stride, gate, out, n, a.W, a.top);
    return tb_launch_status();
}

extern "C" int tb_moe_route(const MoeRouteArgs* args, cudaStream_t stream) {
    const MoeRouteArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.E <= 0 || a.top < 1 || a.top > a.E || a.groups < 1 || a.E % a.groups || a.keep < 1 || a.keep > a.groups ||
        a.group_top < 1 || a.group_top > 8 || a.groups > 1024)
        return tb_refuse("moe_route: experts=%d top=%d groups=%d keep=%d group_top=%d", a.E, a.top, a.groups, a.keep, a.group_top);
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * a.E + a.groups) * sizeof(float);
    if (smem > 48 * 1024) return tb_refuse("moe_route: %d experts are more than one block holds", a.E);
    tb_launch(moe_route_kernel, dim3((a.n_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, a);
    return tb_launch_status();
}

static int moe_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms = n > 0 ? n : 148;
    }
    return sms;
}

extern "C" int tb_moe_gate_up(const MoeExpertArgs* args, int dtype, cudaStream_t stream) {
    const MoeExpertArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.W <= 0 || a.W > 12288 || a.ff <= 0 || a.top <= 0) return tb_refuse("moe: W=%d ff=%d top=%d", a.W, a.ff, a.top);
    const int per = 8 * MV_ROWS;                       // rows a CTA's eight warps take in one round
    // as many CTAs as the device holds at once (four of these an SM), each warp taking the same number of rounds: a
    // CTA's start (the pair's expert, the token's row into shared memory) is then paid once for several rounds, and
    // no second, partly filled wave of CTAs follows the first
    const int pairs = a.n_tokens * a.top, most = (a.ff + per - 1) / per, room = 4 * moe_sm_count();
    const int rounds = ((long long)pairs * most + room - 1) / room;
    int ys = (most + rounds - 1) / rounds;
    if (ys > 64) ys = 64;
    TB_DISPATCH_1(dtype, T, tb_launch(moe_gate_up_kernel<T>, dim3(pairs, ys), dim3(256), (size_t)a.W * sizeof(float), stream, a));
    return tb_launch_status();
}

extern "C" int tb_moe_down(const MoeExpertArgs* args, int dtype, cudaStream_t stream) {
    const MoeExpertArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    const size_t smem = (size_t)a.top * a.ff * sizeof(float);
    if (smem > 200 * 1024) return tb_refuse("moe_down: top=%d x ff=%d activations exceed one block's shared memory", a.top, a.ff);
    if (smem > 48 * 1024) {
        cudaError_t e = dtype == TB_BF16 ? cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                         : cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    const int per = 8 * MV_ROWS;
    const int ys = (a.W + per - 1) / per < 64 ? (a.W + per - 1) / per : 64;
    TB_DISPATCH_1(dtype, T, tb_launch(moe_down_kernel<T>, dim3(a.n_tokens, ys), dim3(256), smem, stream, a));
    return tb_launch_status();
}
