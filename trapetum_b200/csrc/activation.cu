// Gated activation of the feed-forward: out = act(gate) * up.
//
// gelu_tanh(g) = 0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3))), the form the
// reference computes in gelu_mul_k (runtime/cuda/codebook_gemv.cu:531-537); silu
// is there for arrangements that want it (codebook_gemv.cu:205-209).  The input
// holds gate in columns [0, I) and up in [I, 2I) of each row; all math is 32-bit.
//
// clamped_swish is the gate of feed-forwards that bound both branches by a limit L:
//   g' = min(g, L), u' = clamp(u, -L, L), out = g' sigmoid(1.702 g') (u' + 1).
//
// Also here: the per-token gate of a token-indexed side input (tb_token_gate) and the bias row (tb_add_bias).
#include "common.cuh"

TB_EXPORT_ERROR()

#define ACT_GELU_TANH 0
#define ACT_SILU 1
#define ACT_CLAMPED_SWISH 2

__device__ __forceinline__ float gelu_tanh_f(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

template <typename TI, typename TO, int ACT>
__global__ void gated_act_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int inter, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const float g = to_f<TI>(gu[row * 2 * inter + c]);
    const float u = to_f<TI>(gu[row * 2 * inter + inter + c]);
    if (ACT == ACT_CLAMPED_SWISH) {
        const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
        out[row * inter + c] = from_f<TO>(gc / (1.0f + expf(-1.702f * gc)) * (uc + 1.0f));
        return;
    }
    const float a = (ACT == ACT_GELU_TANH) ? gelu_tanh_f(g) : silu_f(g);
    out[row * inter + c] = from_f<TO>(a * u);
}

static int gated_act_launch(const void* gu, int in_dtype, void* out, int out_dtype, int rows, int inter,
                            int act, float limit, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) return tb_refuse("gated_act: intermediate size %d", inter);
    if (act < ACT_GELU_TANH || act > ACT_CLAMPED_SWISH) return tb_refuse("gated_act: unknown activation %d", act);
    dim3 grid(rows, (inter + 255) / 256);
    if (grid.y > 65535) return tb_refuse("gated_act: intermediate size %d is too wide", inter);
#define LAUNCH(TI, TO)                                                                         \
    do {                                                                                       \
        if (act == ACT_GELU_TANH) tb_launch(gated_act_kernel<TI, TO, ACT_GELU_TANH>, dim3(grid), dim3(256), 0, stream, (const TI*)gu, (TO*)out, inter, limit); \
        else if (act == ACT_SILU) tb_launch(gated_act_kernel<TI, TO, ACT_SILU>, dim3(grid), dim3(256), 0, stream, (const TI*)gu, (TO*)out, inter, limit); \
        else tb_launch(gated_act_kernel<TI, TO, ACT_CLAMPED_SWISH>, dim3(grid), dim3(256), 0, stream, (const TI*)gu, (TO*)out, inter, limit); \
    } while (0)
    if (in_dtype == TB_F32 && out_dtype == TB_F32) LAUNCH(float, float);
    else if (in_dtype == TB_F32 && out_dtype == TB_BF16) LAUNCH(float, bf16);
    else if (in_dtype == TB_BF16 && out_dtype == TB_BF16) LAUNCH(bf16, bf16);
    else if (in_dtype == TB_BF16 && out_dtype == TB_F32) LAUNCH(bf16, float);
    else return tb_refuse("gated_act: unknown dtype codes %d %d", in_dtype, out_dtype);
#undef LAUNCH
    return tb_launch_status();
}

extern "C" int tb_gated_act(const void* gu, int in_dtype, void* out, int out_dtype, int rows, int inter,
                            int act, cudaStream_t stream) {
    if (act == ACT_CLAMPED_SWISH) return tb_refuse("gated_act: this activation needs its limit (tb_gated_act_limit)");
    return gated_act_launch(gu, in_dtype, out, out_dtype, rows, inter, act, 0.f, stream);
}

// The same with the activation's parameter (the limit of clamped_swish).
extern "C" int tb_gated_act_limit(const void* gu, int in_dtype, void* out, int out_dtype, int rows, int inter,
                                  int act, float limit, cudaStream_t stream) {
    return gated_act_launch(gu, in_dtype, out, out_dtype, rows, inter, act, limit, stream);
}

// out[t, j] = gelu_tanh(g[t, j]) * table[ids[t], col0 + j]: the gate of a side input that is looked up by token id.
// g may come as n_splits partial sums (the split-K output of its product), added here in split order.
template <typename TI, typename TW, typename TO>
__global__ void token_gate_kernel(const TI* __restrict__ g, int n_splits, long long split_stride, const int* __restrict__ ids,
                                  const TW* __restrict__ table, long long table_stride, int col0, int vocab,
                                  TO* __restrict__ out, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= dim) return;
    const int id = ids[t];
    const float e = (id >= 0 && id < vocab) ? to_f<TW>(table[(size_t)id * table_stride + col0 + j]) : __int_as_float(0x7fc00000);
    float v = to_f<TI>(g[t * dim + j]);
    for (int s0 = 1; s0 < n_splits; s0 += 8) {                      // eight splits requested at a time, added in order
        float p[8];
#pragma unroll
        for (int k = 0; k < 8; k++) p[k] = s0 + k < n_splits ? to_f<TI>(g[(size_t)(s0 + k) * split_stride + t * dim + j]) : 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) if (s0 + k < n_splits) v += p[k];
    }
    out[t * dim + j] = from_f<TO>(gelu_tanh_f(v) * e);
}

extern "C" int tb_token_gate(const void* g, int g_dtype, int n_splits, long long split_stride, const int* ids, const void* table, int table_dtype,
                             long long table_stride, int col0, int vocab, void* out, int out_dtype, int rows, int dim,
                             cudaStream_t stream) {
    if (rows <= 0 || dim <= 0) return 0;
    dim3 grid(rows, (dim + 127) / 128);
    if (grid.y > 65535) return tb_refuse("token_gate: dim %d is too wide", dim);
    if (n_splits < 1) return tb_refuse("token_gate: n_splits=%d", n_splits);
#define LAUNCH(TI, TW, TO) tb_launch(token_gate_kernel<TI, TW, TO>, dim3(grid), dim3(128), 0, stream, (const TI*)g, n_splits, split_stride, ids, \
                                     (const TW*)table, table_stride, col0, vocab, (TO*)out, dim)
#define LAUNCH_O(TI, TW) do { if (out_dtype == TB_F32) LAUNCH(TI, TW, float); else LAUNCH(TI, TW, bf16); } while (0)
    if (out_dtype != TB_F32 && out_dtype != TB_BF16) return tb_refuse("token_gate: unknown output dtype %d", out_dtype);
    if (g_dtype == TB_F32 && table_dtype == TB_F32) LAUNCH_O(float, float);
    else if (g_dtype == TB_F32 && table_dtype == TB_BF16) LAUNCH_O(float, bf16);
    else if (g_dtype == TB_BF16 && table_dtype == TB_BF16) LAUNCH_O(bf16, bf16);
    else if (g_dtype == TB_BF16 && table_dtype == TB_F32) LAUNCH_O(bf16, float);
    else return tb_refuse("token_gate: unknown dtype codes %d %d", g_dtype, table_dtype);
#undef LAUNCH_O
#undef LAUNCH
    return tb_launch_status();
}

// x[r, c] += bias[c] in place, the sum in 32-bit (rows may be wider than `width`: row_stride elements apart).
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ x, long long row_stride, const TB* __restrict__ bias, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    T* p = x + (size_t)blockIdx.x * row_stride + c;
    *p = from_f<T>(to_f<T>(*p) + to_f<TB>(bias[c]));
}

extern "C" int tb_add_bias(void* x, int x_dtype, long long row_stride, const void* bias, int bias_dtype, int rows,
                           int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    dim3 grid(rows, (width + 255) / 256);
    if (grid.y > 65535) return tb_refuse("add_bias: width %d is too wide", width);
#define LAUNCH(T, TB) tb_launch(add_bias_kernel<T, TB>, dim3(grid), dim3(256), 0, stream, (T*)x, row_stride, (const TB*)bias, width)
    if (x_dtype == TB_F32 && bias_dtype == TB_F32) LAUNCH(float, float);
    else if (x_dtype == TB_F32 && bias_dtype == TB_BF16) LAUNCH(float, bf16);
    else if (x_dtype == TB_BF16 && bias_dtype == TB_BF16) LAUNCH(bf16, bf16);
    else if (x_dtype == TB_BF16 && bias_dtype == TB_F32) LAUNCH(bf16, float);
    else return tb_refuse("add_bias: unknown dtype codes %d %d", x_dtype, bias_dtype);
#undef LAUNCH
    return tb_launch_status();
}

// Activation of a feed-forward without a gate branch: out = act(u), act = relu(u)^2 (code 3).  The input is a window of
// `inter` columns, starting at column col0, of a product given as 32-bit partial sums [splits][rows][row_stride]
// (added here in split order), so that one product may carry other columns beside it (a router's logits).
#define ACT_RELU2 3

template <typename TO>
__global__ void unary_act_kernel(const float* __restrict__ part, int n_splits, long long split_stride, long long row_stride,
                                 int col0, TO* __restrict__ out, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const float* p = part + row * row_stride + col0 + c;
    float u = 0.f;
    for (int s = 0; s < n_splits; s++) u += p[(size_t)s * split_stride];
    u = fmaxf(u, 0.f);
    out[row * inter + c] = from_f<TO>(u * u);
}

extern "C" int tb_unary_act(const float* part, int n_splits, long long split_stride, long long row_stride, int col0,
                            void* out, int out_dtype, int rows, int inter, int act, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || n_splits < 1 || col0 < 0) return tb_refuse("unary_act: %d columns from column %d of %d partial sums", inter, col0, n_splits);
    if (act != ACT_RELU2) return tb_refuse("unary_act: unknown activation %d (3: the square of relu)", act);
    dim3 grid(rows, (inter + 255) / 256);
    if (grid.y > 65535) return tb_refuse("unary_act: %d columns are too many", inter);
    TB_DISPATCH_1(out_dtype, T, tb_launch(unary_act_kernel<T>, dim3(grid), dim3(256), 0, stream, part, n_splits, split_stride,
                                          row_stride, col0, (T*)out, inter));
    return tb_launch_status();
}
