// A gated linear recurrence per channel, S_t = a_t S_(t-1) + b_t, with what the real-gated linear
// recurrent unit puts around it.  Everything that enters the recurrence is 32-bit.
//
//   causal_conv_kernel    u[t, c] = bias[c] + sum_k w[c, k] x[t - (taps - 1 - k), c], x = the projection plus
//                         its bias; inputs before the step come from the slot's state (the last taps - 1
//                         inputs of the sequence; zeros before its start).  Output float32.
//   rglru_gate_kernel     from the two gate pre-activations of a channel (a block-diagonal product of u,
//                         made by the grouped product in float32): r = sigmoid(. + bias), i = sigmoid(. + bias),
//                         log a = -c r softplus(lambda), a = exp(log a), b = sqrt(1 - a^2) i u, with
//                         1 - a^2 = -expm1(2 log a).  a and b overwrite the pre-activations.
//   linear_scan_kernel    a thread per (sequence, channel) walks the step's tokens from the slot's state,
//                         writes out[t, c] = S_t * gelu_tanh(y[t, c] + bias) in the compute dtype, leaves
//                         the state updated and moves the convolution's inputs on.  Long prompts are cut into
//                         chunks that run side by side (two passes and a carry between them).
//
// State of a slot: float32 [width] S, then [taps - 1][width] the convolution's last inputs, oldest first.
// ExiledOfCode/KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106).
#include "common.cuh"

namespace kl {

constexpr int LR_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ proj, long long ld, int x_col, const float* __restrict__ x_bias,
                   const float* __restrict__ w, const float* __restrict__ bias, int taps,
                   const float* __restrict__ state, long long state_ld, const int* __restrict__ cu_tokens,
                   const int* __restrict__ seq_slots, const int* __restrict__ seq_new, int width, float* __restrict__ u) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y, l = blockIdx.x;
    if (l >= seq_new[s]) return;
    const int row0 = cu_tokens[s], slot = seq_slots[s];
    if (slot < 0) return;
    const float* tail = state + (size_t)slot * state_ld + width;            // [taps - 1][width]
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = bias ? bias[c] : 0.f;
        const float xb = x_bias ? x_bias[c] : 0.f;
        for (int k = 0; k < taps; ++k) {
            const int li = l - (taps - 1 - k);
            const float x = li >= 0 ? to_f32(proj[(size_t)(row0 + li) * ld + x_col + c]) + xb
                                    : tail[(size_t)(taps - 1 + li) * width + c];
            acc = fmaf(w[(size_t)c * taps + k], x, acc);
        }
        u[(size_t)(row0 + l) * width + c] = acc;
    }
}

__global__ void __launch_bounds__(256)
rglru_gate_kernel(float* __restrict__ gates, const float* __restrict__ u, const float* __restrict__ r_bias,
                  const float* __restrict__ i_bias, const float* __restrict__ softplus_lambda, float decay_scale,
                  int tokens, int width, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)tokens * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width;
        const int c = (int)(idx - t * width);
        const int b = c / block, j = c - b * block;
        float* g = gates + t * 2 * (size_t)width + (size_t)b * 2 * block;
        const float r = 1.0f / (1.0f + expf(-(g[j] + r_bias[c])));
        const float i = 1.0f / (1.0f + expf(-(g[block + j] + i_bias[c])));
        const float log_a = -decay_scale * r * softplus_lambda[c];
        g[j] = expf(log_a);
        g[block + j] = sqrtf(-expm1f(2.0f * log_a)) * i * u[idx];
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The convolution's inputs move on: the last taps - 1 inputs of the sequence, oldest first.
template <typename T>
__device__ __forceinline__ void move_taps(float* __restrict__ tail, const T* __restrict__ proj, long long ld, int x_col,
                                          const float* __restrict__ x_bias, int taps, int row0, int n, int width, int c) {
    if (taps <= 1) return;
    const float xb = x_bias ? x_bias[c] : 0.f;
    float keep[LR_MAX_TAPS];
#pragma unroll
    for (int q = 0; q < LR_MAX_TAPS; ++q) {
        if (q < taps - 1) {
            const int li = n - (taps - 1) + q;                     // the input that lands at place q
            keep[q] = li >= 0 ? to_f32(proj[(size_t)(row0 + li) * ld + x_col + c]) + xb : tail[(size_t)(q + n) * width + c];
        }
    }
#pragma unroll
    for (int q = 0; q < LR_MAX_TAPS; ++q)
        if (q < taps - 1) tail[(size_t)q * width + c] = keep[q];
}

// MODE 0: a thread walks all of its sequence's tokens from the slot's state and leaves the state updated.
// Long prompts take three launches instead, over chunks of `chunk` tokens (blockIdx.y): MODE 1 leaves every chunk's
// (product of a, result from zero) in scratch [sequences][chunks][2][width]; linear_carry_kernel walks the chunks,
// puts every chunk's starting state where its product was and updates the slot's state; MODE 2 walks every chunk
// again from its starting state and writes the outputs.
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const float* __restrict__ gates, int block, const T* __restrict__ proj, long long ld, int y_col, int x_col,
                   const float* __restrict__ y_bias, const float* __restrict__ x_bias, int taps, float* __restrict__ state,
                   long long state_ld, const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots,
                   const int* __restrict__ seq_new, int width, T* __restrict__ out, float* __restrict__ scratch, int chunk) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.z;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = seq_slots[s];
    if (c >= width || slot < 0) return;
    const int row0 = cu_tokens[s], n = seq_new[s];
    const int l0 = MODE == 0 ? 0 : blockIdx.y * chunk, l1 = MODE == 0 ? n : min(n, l0 + chunk);
    if (l0 >= n) return;
    const int b = c / block, j = c - b * block;
    float* st = state + (size_t)slot * state_ld;
    float* sc = MODE == 0 ? nullptr : scratch + ((size_t)s * gridDim.y + blockIdx.y) * 2 * width;
    float S = MODE == 0 ? st[c] : (MODE == 1 ? 0.f : sc[c]);
    float P = 1.f;
    const float yb = y_bias ? y_bias[c] : 0.f;
    const float* g = gates + (size_t)row0 * 2 * width + (size_t)b * 2 * block + j;
    const T* y = proj + (size_t)row0 * ld + y_col + c;
    T* o = out + (size_t)row0 * width + c;
#pragma unroll 4
    for (int l = l0; l < l1; ++l) {
        const float a = g[(size_t)l * 2 * width], bx = g[(size_t)l * 2 * width + block];
        S = fmaf(a, S, bx);
        if (MODE == 1) P *= a;
        else o[(size_t)l * width] = from_f32<T>(S * gelu_tanh_f(to_f32(y[(size_t)l * ld]) + yb));
    }
    if (MODE == 1) { sc[c] = P; sc[width + c] = S; }
    if (MODE == 0) {
        st[c] = S;
        move_taps(st + width, proj, ld, x_col, x_bias, taps, row0, n, width, c);
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
linear_carry_kernel(float* __restrict__ scratch, int chunks, int chunk, const T* __restrict__ proj, long long ld, int x_col,
                    const float* __restrict__ x_bias, int taps, float* __restrict__ state, long long state_ld,
                    const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots, const int* __restrict__ seq_new, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = seq_slots[s];
    if (c >= width || slot < 0) return;
    const int n = seq_new[s];
    float* st = state + (size_t)slot * state_ld;
    float S = st[c];
    for (int k = 0; k * chunk < n; ++k) {
        float* sc = scratch + ((size_t)s * chunks + k) * 2 * width;
        const float P = sc[c], B = sc[width + c];
        sc[c] = S;
        S = fmaf(P, S, B);
    }
    st[c] = S;
    move_taps(st + width, proj, ld, x_col, x_bias, taps, cu_tokens[s], n, width, c);
}

}  // namespace kl

using namespace kl;

KL_API int kl_causal_conv(const void* proj, long long ld, int x_col, const float* x_bias, const float* w, const float* bias, int taps,
                          const float* state, long long state_ld, const int* cu_tokens, const int* seq_slots, const int* seq_new,
                          int n_seqs, int max_new, int width, float* u, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (taps < 1 || taps > LR_MAX_TAPS || width <= 0 || n_seqs > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid(max_new, n_seqs);
    const int threads = width >= 256 ? 256 : (width + 31) / 32 * 32;
    if (dtype == KL_F32)
        launch_kernel(causal_conv_kernel<float>, grid, threads, 0, stream, (const float*)proj, ld, x_col, x_bias, w, bias, taps, state,
                      state_ld, cu_tokens, seq_slots, seq_new, width, u);
    else if (dtype == KL_BF16)
        launch_kernel(causal_conv_kernel<bf16>, grid, threads, 0, stream, (const bf16*)proj, ld, x_col, x_bias, w, bias, taps, state,
                      state_ld, cu_tokens, seq_slots, seq_new, width, u);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

KL_API int kl_rglru_gate(float* gates, const float* u, const float* r_bias, const float* i_bias, const float* softplus_lambda,
                         float decay_scale, int tokens, int width, int block, cudaStream_t stream) {
    if (tokens <= 0) return KL_OK;
    if (width <= 0 || block <= 0 || width % block) return KL_ERR_BAD_SIZE;
    const int blocks = kl::strided_grid((size_t)tokens * width, 256, 16);
    launch_kernel(rglru_gate_kernel, blocks, 256, 0, stream, gates, u, r_bias, i_bias, softplus_lambda, decay_scale, tokens, width, block);
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// scratch: null (a thread per sequence and channel walks the whole step), or float32 [n_seqs][ceil(max_new / chunk)][2][width]
// for the three launches over chunks of `chunk` tokens.
KL_API int kl_linear_scan(const float* gates, int block, const void* proj, long long ld, int y_col, int x_col, const float* y_bias,
                          const float* x_bias, int taps, float* state, long long state_ld, const int* cu_tokens,
                          const int* seq_slots, const int* seq_new, int n_seqs, int max_new, int width, void* out, float* scratch,
                          int chunk, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0) return KL_OK;
    if (taps < 1 || taps > LR_MAX_TAPS || width <= 0 || block <= 0 || width % block || n_seqs > 65535) return KL_ERR_BAD_SIZE;
    if (dtype != KL_F32 && dtype != KL_BF16) return KL_ERR_BAD_DTYPE;
    if (scratch != nullptr && (chunk <= 0 || max_new <= 0)) return KL_ERR_BAD_SIZE;
    const int chunks = scratch ? (max_new + chunk - 1) / chunk : 1;
    if (chunks > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid((width + 127) / 128, chunks, n_seqs);
#define KL_SCAN(T, MODE)                                                                                                    \
    launch_kernel(linear_scan_kernel<T, MODE>, grid, 128, 0, stream, gates, block, (const T*)proj, ld, y_col, x_col, y_bias, x_bias, \
                  taps, state, state_ld, cu_tokens, seq_slots, seq_new, width, (T*)out, scratch, chunk)
#define KL_CARRY(T)                                                                                                         \
    launch_kernel(linear_carry_kernel<T>, dim3((width + 127) / 128, n_seqs), 128, 0, stream, scratch, chunks, chunk, (const T*)proj, ld, \
                  x_col, x_bias, taps, state, state_ld, cu_tokens, seq_slots, seq_new, width)
    if (scratch == nullptr) {
        if (dtype == KL_F32) KL_SCAN(float, 0); else KL_SCAN(bf16, 0);
    } else if (dtype == KL_F32) {
        KL_SCAN(float, 1); KL_LAUNCH_CHECK(); KL_CARRY(float); KL_LAUNCH_CHECK(); KL_SCAN(float, 2);
    } else {
        KL_SCAN(bf16, 1); KL_LAUNCH_CHECK(); KL_CARRY(bf16); KL_LAUNCH_CHECK(); KL_SCAN(bf16, 2);
    }
#undef KL_SCAN
#undef KL_CARRY
    KL_LAUNCH_CHECK();
    return KL_OK;
}
