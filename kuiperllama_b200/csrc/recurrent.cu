// Recurrent mixers: state of a fixed size per sequence instead of keys and values per token.
//
// * minGRU: s_t = (1 - z_t) s_(t-1) + z_t c_t per channel, the gates a function of the current
//   token alone.
// * Gated delta rule: per head a matrix S (key size x value size) with
//       S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//   after a short causal convolution and SiLU on q, k, v and unit-length q and k.
//
// Both run over a ragged batch (sequence i owns rows cu_tokens[i] .. cu_tokens[i + 1] of the step,
// in time order) from the state that the cache keeps per slot, and leave the state after the
// step's last token there: a prompt in one step, in pieces, or token by token gives the same
// sums in the same order.  State, gates, decays and unit norms are 32-bit; the projections come
// in the compute dtype as column slices of one stacked product (row stride `ld`).
// ExiledOfCode/KuiperLLama has no recurrent mixer; its one sequence-mixing op is attention over
// a cache (mha_kernel.cu:61,74-106).
#include "common.cuh"

namespace kl {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------------------------------ minGRU
// One thread per (sequence, channel).  z = sigmoid(pz + bz); u = px + bx; candidate c = u + 1/2
// for u >= 0, sigmoid(u) below; out = s_t * silu(pg).
template <typename T>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(const T* __restrict__ proj, long long ld, int z_col, int x_col, int g_col, const float* __restrict__ bz,
                   const float* __restrict__ bx, float* __restrict__ state, long long state_ld, T* __restrict__ out,
                   const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int s = blockIdx.y;
    const int r0 = cu_tokens[s], r1 = cu_tokens[s + 1];
    if (r1 <= r0) return;
    float* st = state + (size_t)seq_slots[s] * state_ld + c;
    float S = *st;
    const float biasz = bz ? bz[c] : 0.f, biasx = bx ? bx[c] : 0.f;
    constexpr int U = 4;                                  // rows whose loads are in flight together
    for (int r = r0; r < r1; r += U) {
        float pz[U], px[U], pg[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const bool ok = r + k < r1;
            const T* row = proj + (size_t)(ok ? r + k : r) * ld;
            pz[k] = to_f32(row[z_col + c]);
            px[k] = to_f32(row[x_col + c]);
            pg[k] = to_f32(row[g_col + c]);
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (r + k < r1) {
                const float z = sigmoidf_(pz[k] + biasz);
                const float u = px[k] + biasx;
                const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
                S = (1.0f - z) * S + z * cand;
                const float g = pg[k];
                out[(size_t)(r + k) * width + c] = from_f32<T>(S * (g * sigmoidf_(g)));
            }
        }
    }
    *st = S;
}

// The same recurrence for steps with long sequences, in three passes over chunks of MG_CHUNK tokens
// (s_t = a_t s_(t-1) + b_t with a = 1 - z, b = z c composes: a chunk maps its incoming state s to
// A s + B).  Pass 1, a thread per (chunk, channel): A and B of the chunk.  Pass 2, a thread per
// (sequence, channel): the state at the start of every chunk, chunk after chunk, and the slot's state
// after the step.  Pass 3, a thread per (chunk, channel): the chunk again from its true start, writing
// out.  Chunks are counted per sequence from the step's first token; chunk c of sequence s is entry
// chunk_first[s] + c of the (A, B) arrays, which the host sizes for the step.
constexpr int MG_CHUNK = 64;

template <typename T>
__device__ __forceinline__ void mingru_gates(const T* __restrict__ row, int z_col, int x_col, int c, float biasz, float biasx,
                                             float& a, float& b) {
    const float z = sigmoidf_(to_f32(row[z_col + c]) + biasz);
    const float u = to_f32(row[x_col + c]) + biasx;
    a = 1.0f - z;
    b = z * (u >= 0.f ? u + 0.5f : sigmoidf_(u));
}

template <typename T, int PASS>
__global__ void __launch_bounds__(128)
mingru_chunk_kernel(const T* __restrict__ proj, long long ld, int z_col, int x_col, int g_col, const float* __restrict__ bz,
                    const float* __restrict__ bx, float* __restrict__ state, long long state_ld, T* __restrict__ out,
                    float* __restrict__ AB, const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots, int width,
                    int max_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int s = blockIdx.z;
    const int r0 = cu_tokens[s], r1 = cu_tokens[s + 1];
    const int n_chunks = (r1 - r0 + MG_CHUNK - 1) / MG_CHUNK;
    const float biasz = bz ? bz[c] : 0.f, biasx = bx ? bx[c] : 0.f;
    // (A, B, start state) of chunk k of sequence s: three floats per channel at entry s * max_chunks + k
    float* ab = AB + ((size_t)s * max_chunks) * 3 * width + c;
    if (PASS == 2) {
        float* st = state + (size_t)seq_slots[s] * state_ld + c;
        float S = *st;
        for (int k = 0; k < n_chunks; ++k) {
            float* e = ab + (size_t)k * 3 * width;
            e[2 * width] = S;
            S = fmaf(e[0], S, e[width]);
        }
        if (n_chunks > 0) *st = S;
        return;
    }
    const int k = blockIdx.y;
    if (k >= n_chunks) return;
    float* e = ab + (size_t)k * 3 * width;
    const int t0 = r0 + k * MG_CHUNK, t1 = min(t0 + MG_CHUNK, r1);
    if (PASS == 1) {
        float A = 1.f, B = 0.f;
        for (int r = t0; r < t1; ++r) {
            float a, b;
            mingru_gates(proj + (size_t)r * ld, z_col, x_col, c, biasz, biasx, a, b);
            A *= a;
            B = fmaf(a, B, b);
        }
        e[0] = A;
        e[width] = B;
    } else {
        float S = e[2 * width];
        for (int r = t0; r < t1; ++r) {
            const T* row = proj + (size_t)r * ld;
            float a, b;
            mingru_gates(row, z_col, x_col, c, biasz, biasx, a, b);
            S = fmaf(a, S, b);
            const float g = to_f32(row[g_col + c]);
            out[(size_t)r * width + c] = from_f32<T>(S * (g * sigmoidf_(g)));
        }
    }
}

// ------------------------------------------------------------------------------------------ gated delta rule
// Step 1, one CTA per token: the short convolution and SiLU over the C = 2 G d + H dv channels of
// q | k | v, unit length for each q and k head (q also times q_scale), and the token's beta and
// decay per head.  The taps before the step's first token come from the slot's convolution state
// ([taps - 1][C], entry m holding the input of time m - (taps - 1) relative to the step's start).
//   prep [rows][C] float32: q | k | v after all that;  bg [rows][2 H]: beta | decay.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, long long ld, int conv_col, int b_col, int a_col,
                     const float* __restrict__ taps_w, int taps, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                     const float* __restrict__ state, long long state_ld, long long conv_off,
                     float* __restrict__ prep, float* __restrict__ bg, const int* __restrict__ cu_tokens,
                     const int* __restrict__ seq_slots, int H, int G, int d, int dv, float q_scale, float unit_eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float buf[];                        // [C]
    const int s = blockIdx.y, j = blockIdx.x;
    const int r0 = cu_tokens[s];
    if (j >= cu_tokens[s + 1] - r0) return;
    const int row = r0 + j;
    const int C = 2 * G * d + H * dv;
    const float* cs = state + (size_t)seq_slots[s] * state_ld + conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int i = 0; i < taps; ++i) {
            const int tt = j - (taps - 1 - i);
            const float x = tt >= 0 ? to_f32(proj[(size_t)(r0 + tt) * ld + conv_col + c]) : cs[(size_t)(taps - 1 + tt) * C + c];
            acc = fmaf(taps_w[(size_t)c * taps + i], x, acc);
        }
        buf[c] = acc * sigmoidf_(acc);
    }
    __syncthreads();
    float* o = prep + (size_t)row * C;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int seg = warp; seg < 2 * G; seg += nwarps) {    // q heads, then k heads
        const float* x = buf + (size_t)seg * d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
        ss = warp_sum(ss);
        const float inv = (seg < G ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        for (int i = lane; i < d; i += 32) o[(size_t)seg * d + i] = x[i] * inv;
    }
    for (int c = 2 * G * d + threadIdx.x; c < C; c += blockDim.x) o[c] = buf[c];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const T* pr = proj + (size_t)row * ld;
        bg[(size_t)row * 2 * H + h] = sigmoidf_(to_f32(pr[b_col + h]));
        bg[(size_t)row * 2 * H + H + h] = expf(-expf(A_log[h]) * softplusf_(to_f32(pr[a_col + h]) + dt_bias[h]));
    }
}

// Step 2, the recurrence.  A column j of S (all keys' weights for value element j) never meets
// another column, so a CTA owns some columns of one head of one sequence and walks the tokens in
// order.  A column is cut over LPC adjacent lanes of 32 key elements each (d <= 32 LPC), kept in
// registers; the tokens' k, q, v, beta and decay come through shared memory a tile of tokens at a time.
// The read-out after the write, o = S_new^T q, is taken from the state before it:
//     S_new^T q = g S^T q + (k . q) u,
// so that both products with the old state (S^T k and S^T q) run side by side and only one
// multiply-add per element lies between one token's products and the next one's.
// Before it starts, the first CTA of a sequence moves the convolution state on (the raw projections
// of the step's last taps - 1 tokens; step 1 has finished with the old one).
constexpr int DR_THREADS = 128, DR_TILE = 8, DR_DPT = 32;

template <typename T, int LPC>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ prep, const float* __restrict__ bg, const T* __restrict__ proj, long long ld,
                  int conv_col, int taps, float* __restrict__ state, long long state_ld, long long conv_off,
                  float* __restrict__ out, const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots,
                  int H, int G, int d, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int COLS = DR_THREADS / LPC;
    constexpr int DP = DR_DPT * LPC;                      // padded key size
    constexpr int DPS = (DR_DPT + 1) * LPC;               // in shared memory every part starts one bank further on
    __shared__ float ks[DR_TILE][DPS], qs[DR_TILE][DPS], vs[DR_TILE][COLS], bs[DR_TILE], gs[DR_TILE], kqs[DR_TILE];
    const int s = blockIdx.z, h = blockIdx.y;
    const int r0 = cu_tokens[s], r1 = cu_tokens[s + 1];
    if (r1 <= r0) return;
    const int slot = seq_slots[s];
    const int C = 2 * G * d + H * dv;
    float* slot_state = state + (size_t)slot * state_ld;
    if (blockIdx.x == 0 && h == 0 && taps > 1) {
        float* cs = slot_state + conv_off;
        const int n_new = r1 - r0;
        for (int c = threadIdx.x; c < C; c += blockDim.x)
            for (int m = 0; m < taps - 1; ++m) {          // ascending: an old entry is read before it is overwritten
                const int tt = n_new - (taps - 1) + m;
                cs[(size_t)m * C + c] = tt >= 0 ? to_f32(proj[(size_t)(r0 + tt) * ld + conv_col + c]) : cs[(size_t)(n_new + m) * C + c];
            }
    }
    const int g = h / (H / G);
    const int part = threadIdx.x % LPC, col_local = threadIdx.x / LPC;
    const int col = blockIdx.x * COLS + col_local;
    const bool live = col < dv;
    float S[DR_DPT];
    float* sp = slot_state + ((size_t)h * dv + (live ? col : 0)) * d + part * DR_DPT;
#pragma unroll
    for (int i = 0; i < DR_DPT; ++i) S[i] = (live && part * DR_DPT + i < d) ? sp[i] : 0.f;

    for (int t0 = r0; t0 < r1; t0 += DR_TILE) {
        const int nt = min(DR_TILE, r1 - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < nt * DP; e += blockDim.x) {
            const int tt = e / DP, i = e - tt * DP;
            const float* p = prep + (size_t)(t0 + tt) * C;
            const int at = i + i / DR_DPT;
            ks[tt][at] = i < d ? p[(size_t)(G + g) * d + i] : 0.f;
            qs[tt][at] = i < d ? p[(size_t)g * d + i] : 0.f;
        }
        for (int e = threadIdx.x; e < nt * COLS; e += blockDim.x) {
            const int tt = e / COLS, c = e - tt * COLS;
            const int cc = blockIdx.x * COLS + c;
            vs[tt][c] = cc < dv ? prep[(size_t)(t0 + tt) * C + 2 * G * d + (size_t)h * dv + cc] : 0.f;
        }
        if (threadIdx.x < nt) {
            bs[threadIdx.x] = bg[(size_t)(t0 + threadIdx.x) * 2 * H + h];
            gs[threadIdx.x] = bg[(size_t)(t0 + threadIdx.x) * 2 * H + H + h];
        }
        {                                                  // k . q of every token of the tile, a warp each
            const int lane = threadIdx.x & 31;
            for (int tt = threadIdx.x >> 5; tt < nt; tt += DR_THREADS / 32) {
                const float* p = prep + (size_t)(t0 + tt) * C;
                float a = 0.f;
                for (int i = lane; i < d; i += 32) a = fmaf(p[(size_t)(G + g) * d + i], p[(size_t)g * d + i], a);
                a = warp_sum(a);
                if (lane == 0) kqs[tt] = a;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* kk = &ks[tt][part * (DR_DPT + 1)];
            const float* qq = &qs[tt][part * (DR_DPT + 1)];
            const float decay = gs[tt], beta = bs[tt];
            float sk[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < DR_DPT; ++i) {
                sk[i & 3] = fmaf(S[i], kk[i], sk[i & 3]);
                sq[i & 3] = fmaf(S[i], qq[i], sq[i & 3]);
            }
            float skt = (sk[0] + sk[1]) + (sk[2] + sk[3]), sqt = (sq[0] + sq[1]) + (sq[2] + sq[3]);
#pragma unroll
            for (int o = LPC >> 1; o > 0; o >>= 1) {
                skt += __shfl_xor_sync(0xffffffffu, skt, o);
                sqt += __shfl_xor_sync(0xffffffffu, sqt, o);
            }
            const float u = beta * (vs[tt][col_local] - decay * skt);
#pragma unroll
            for (int i = 0; i < DR_DPT; ++i) S[i] = fmaf(kk[i], u, decay * S[i]);
            if (live && part == 0) out[((size_t)(t0 + tt) * H + h) * dv + col] = fmaf(kqs[tt], u, decay * sqt);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DR_DPT; ++i)
            if (part * DR_DPT + i < d) sp[i] = S[i];
    }
}

}  // namespace kl

using namespace kl;

// proj: compute dtype [rows, ld]; z, x, g at columns z_col, x_col, g_col (width each); out [rows, width].
// max_new: no sequence brings more rows.  With `chunk_scratch` (float32 [n_seqs * ceil(max_new / 64) * 3 * width]) and a step
// long enough to gain from it, the three-pass chunked form runs (3 launches), else one thread walks each channel.
KL_API int kl_mingru_chunk_tokens() { return MG_CHUNK; }

KL_API int kl_mingru_scan(const void* proj, long long ld, int z_col, int x_col, int g_col, const float* bz, const float* bx,
                          float* state, long long state_ld, void* out, const int* cu_tokens, const int* seq_slots, int n_seqs,
                          int max_new, float* chunk_scratch, int width, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || width <= 0) return KL_OK;
    if (n_seqs > 65535) return KL_ERR_BAD_SIZE;
    if (chunk_scratch != nullptr) {
        const int max_chunks = (max_new + MG_CHUNK - 1) / MG_CHUNK;
        if (max_chunks > 65535) return KL_ERR_BAD_SIZE;
        const dim3 g13((width + 127) / 128, max_chunks, n_seqs), g2((width + 127) / 128, 1, n_seqs);
#define KL_MG(T, PASS, GRID)                                                                                                      \
        launch_kernel(mingru_chunk_kernel<T, PASS>, GRID, 128, 0, stream, (const T*)proj, ld, z_col, x_col, g_col, bz, bx, state, state_ld, \
                      (T*)out, chunk_scratch, cu_tokens, seq_slots, width, max_chunks)
        if (dtype == KL_F32) { KL_MG(float, 1, g13); KL_MG(float, 2, g2); KL_MG(float, 3, g13); }
        else if (dtype == KL_BF16) { KL_MG(bf16, 1, g13); KL_MG(bf16, 2, g2); KL_MG(bf16, 3, g13); }
        else return KL_ERR_BAD_DTYPE;
#undef KL_MG
        KL_LAUNCH_CHECK();
        return KL_OK;
    }
    const dim3 grid((width + 127) / 128, n_seqs);
    if (dtype == KL_F32)
        launch_kernel(mingru_scan_kernel<float>, grid, 128, 0, stream, (const float*)proj, ld, z_col, x_col, g_col, bz, bx, state, state_ld,
                      (float*)out, cu_tokens, seq_slots, width);
    else if (dtype == KL_BF16)
        launch_kernel(mingru_scan_kernel<bf16>, grid, 128, 0, stream, (const bf16*)proj, ld, z_col, x_col, g_col, bz, bx, state, state_ld,
                      (bf16*)out, cu_tokens, seq_slots, width);
    else
        return KL_ERR_BAD_DTYPE;
    KL_LAUNCH_CHECK();
    return KL_OK;
}

// The two steps of the gated delta rule.  proj: compute dtype [rows, ld] with q | k | v at conv_col
// (C = 2 G d + H dv columns), beta's and the decay's projections at b_col and a_col (H each).
// state: float32 [slots][state_ld]: S as [H][dv][d] at 0, the convolution state [taps - 1][C] at conv_off.
// prep [rows, C], bg [rows, 2 H], out [rows, H * dv]: float32.  max_new: no sequence brings more rows.
KL_API int kl_gated_delta_rule(const void* proj, long long ld, int conv_col, int b_col, int a_col, const float* taps_w, int taps,
                               const float* A_log, const float* dt_bias, float* state, long long state_ld, long long conv_off,
                               float* prep, float* bg, float* out, const int* cu_tokens, const int* seq_slots, int n_seqs,
                               int max_new, int H, int G, int d, int dv, float q_scale, float unit_eps, int dtype,
                               cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || taps < 1 || d > DR_DPT * 8 || n_seqs > 65535) return KL_ERR_BAD_SIZE;
    const int C = 2 * G * d + H * dv;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return KL_ERR_BAD_SIZE;
    const int lpc = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8;
    const dim3 grid1(max_new, n_seqs);
    const dim3 grid2((dv + DR_THREADS / lpc - 1) / (DR_THREADS / lpc), H, n_seqs);
#define KL_DELTA(T)                                                                                                          \
    do {                                                                                                                     \
        if (smem > 48 * 1024) KL_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        launch_kernel(delta_prepare_kernel<T>, grid1, 256, smem, stream, (const T*)proj, ld, conv_col, b_col, a_col, taps_w, taps, A_log, \
                      dt_bias, (const float*)state, state_ld, conv_off, prep, bg, cu_tokens, seq_slots, H, G, d, dv, q_scale, unit_eps); \
        KL_LAUNCH_CHECK();                                                                                                   \
        if (lpc == 1) launch_kernel(delta_rule_kernel<T, 1>, grid2, DR_THREADS, 0, stream, (const float*)prep, (const float*)bg, (const T*)proj, ld, conv_col, taps, state, state_ld, conv_off, out, cu_tokens, seq_slots, H, G, d, dv); \
        else if (lpc == 2) launch_kernel(delta_rule_kernel<T, 2>, grid2, DR_THREADS, 0, stream, (const float*)prep, (const float*)bg, (const T*)proj, ld, conv_col, taps, state, state_ld, conv_off, out, cu_tokens, seq_slots, H, G, d, dv); \
        else if (lpc == 4) launch_kernel(delta_rule_kernel<T, 4>, grid2, DR_THREADS, 0, stream, (const float*)prep, (const float*)bg, (const T*)proj, ld, conv_col, taps, state, state_ld, conv_off, out, cu_tokens, seq_slots, H, G, d, dv); \
        else launch_kernel(delta_rule_kernel<T, 8>, grid2, DR_THREADS, 0, stream, (const float*)prep, (const float*)bg, (const T*)proj, ld, conv_col, taps, state, state_ld, conv_off, out, cu_tokens, seq_slots, H, G, d, dv); \
    } while (0)
    if (dtype == KL_F32) KL_DELTA(float);
    else if (dtype == KL_BF16) KL_DELTA(bf16);
    else return KL_ERR_BAD_DTYPE;
#undef KL_DELTA
    KL_LAUNCH_CHECK();
    return KL_OK;
}
