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
constexpr int MG_CHUNK = 32;

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
        constexpr int U2 = 8;                             // chunks whose (A, B) are in flight together
        for (int k0 = 0; k0 < n_chunks; k0 += U2) {
            float A[U2], B[U2];
#pragma unroll
            for (int k = 0; k < U2; ++k) {
                const float* e = ab + (size_t)min(k0 + k, n_chunks - 1) * 3 * width;
                A[k] = e[0];
                B[k] = e[width];
            }
#pragma unroll
            for (int k = 0; k < U2; ++k) {
                if (k0 + k < n_chunks) {
                    ab[(size_t)(k0 + k) * 3 * width + 2 * width] = S;
                    S = fmaf(A[k], S, B[k]);
                }
            }
        }
        if (n_chunks > 0) *st = S;
        return;
    }
    const int k = blockIdx.y;
    if (k >= n_chunks) return;
    float* e = ab + (size_t)k * 3 * width;
    const int t0 = r0 + k * MG_CHUNK, t1 = min(t0 + MG_CHUNK, r1);
    constexpr int U = 8;                                  // rows whose loads are in flight together
    float A = 1.f, B = 0.f, S = PASS == 3 ? e[2 * width] : 0.f;
    for (int r = t0; r < t1; r += U) {
        T pz[U], px[U], pg[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const T* row = proj + (size_t)min(r + k, t1 - 1) * ld;
            pz[k] = row[z_col + c];
            px[k] = row[x_col + c];
            if (PASS == 3) pg[k] = row[g_col + c];
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (r + k < t1) {
                const float z = sigmoidf_(to_f32(pz[k]) + biasz);
                const float u = to_f32(px[k]) + biasx;
                const float a = 1.0f - z, b = z * (u >= 0.f ? u + 0.5f : sigmoidf_(u));
                if (PASS == 1) {
                    A *= a;
                    B = fmaf(a, B, b);
                } else {
                    S = fmaf(a, S, b);
                    const float g = to_f32(pg[k]);
                    out[(size_t)(r + k) * width + c] = from_f32<T>(S * (g * sigmoidf_(g)));
                }
            }
        }
    }
    if (PASS == 1) {
        e[0] = A;
        e[width] = B;
    }
}

// ------------------------------------------------------------------------------------------ gated delta rule
// Step 1, one CTA per (token or few tokens, item): an item is a key head g (the short convolution and SiLU over the
// channels of q_g and k_g, unit length for both, q also times q_scale, and k_g . q_g) or a value head h
// (convolution and SiLU over its dv channels, and the token's beta and decay for that head).  The taps
// before the step's first token come from the slot's convolution state ([taps - 1][C], C = 2 G d + H dv,
// entry m holding the input of time m - (taps - 1) relative to the step's start).
//   prep [rows][C] float32: q | k | v after all that;  bg [rows][2 H + G]: beta | decay | k . q.
constexpr int DP_THREADS = 128;

template <typename T>
__device__ __forceinline__ float conv_silu(const T* __restrict__ proj, long long ld, int conv_col, const float* __restrict__ taps_w,
                                           int taps, const float* __restrict__ cs, int C, int r0, int j, int c) {
    float acc = 0.f;
    for (int i = 0; i < taps; ++i) {
        const int tt = j - (taps - 1 - i);
        const float x = tt >= 0 ? to_f32(proj[(size_t)(r0 + tt) * ld + conv_col + c]) : cs[(size_t)(taps - 1 + tt) * C + c];
        acc = fmaf(taps_w[(size_t)c * taps + i], x, acc);
    }
    return acc * sigmoidf_(acc);
}

template <typename T>
__global__ void __launch_bounds__(DP_THREADS)
delta_prepare_kernel(const T* __restrict__ proj, long long ld, int conv_col, int b_col, int a_col,
                     const float* __restrict__ taps_w, int taps, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                     const float* __restrict__ state, long long state_ld, long long conv_off,
                     float* __restrict__ prep, float* __restrict__ bg, const int* __restrict__ cu_tokens,
                     const int* __restrict__ seq_slots, int H, int G, int d, int dv, float q_scale, float unit_eps,
                     int tokens_per_cta) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float buf[];                        // [2 d] and 33 for the sums
    const int s = blockIdx.y, item = blockIdx.z;
    const int r0 = cu_tokens[s];
    const int n_new = cu_tokens[s + 1] - r0;
    const int C = 2 * G * d + H * dv;
    const float* cs = state + (size_t)seq_slots[s] * state_ld + conv_off;
  for (int j = blockIdx.x * tokens_per_cta; j < min((int)(blockIdx.x + 1) * tokens_per_cta, n_new); ++j) {     // a few tokens per CTA in long steps
    const int row = r0 + j;
    float* o = prep + (size_t)row * C;
    float* b = bg + (size_t)row * (2 * H + G);
    if (item >= G) {
        const int h = item - G;
        for (int e = threadIdx.x; e < dv; e += blockDim.x) {
            const int c = 2 * G * d + h * dv + e;
            o[c] = conv_silu(proj, ld, conv_col, taps_w, taps, cs, C, r0, j, c);
        }
        if (threadIdx.x == 0) {
            const T* pr = proj + (size_t)row * ld;
            b[h] = sigmoidf_(to_f32(pr[b_col + h]));
            b[H + h] = expf(-expf(A_log[h]) * softplusf_(to_f32(pr[a_col + h]) + dt_bias[h]));
        }
        continue;
    }
    const int g = item;
    float* scratch = buf + 2 * d;
    float ssq = 0.f, ssk = 0.f;
    for (int e = threadIdx.x; e < 2 * d; e += blockDim.x) {
        const int c = e < d ? g * d + e : (G + g) * d + (e - d);
        const float y = conv_silu(proj, ld, conv_col, taps_w, taps, cs, C, r0, j, c);
        buf[e] = y;
        if (e < d) ssq += y * y; else ssk += y * y;
    }
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
    float kq = 0.f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) kq = fmaf(buf[e], buf[d + e], kq);
    kq = block_sum(kq, scratch);
    const float invq = q_scale / sqrtf(ssq + unit_eps), invk = 1.0f / sqrtf(ssk + unit_eps);
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        o[(size_t)g * d + e] = buf[e] * invq;
        o[(size_t)(G + g) * d + e] = buf[d + e] * invk;
    }
    if (threadIdx.x == 0) b[2 * H + g] = kq * invq * invk;
    __syncthreads();                                      // buf is written again for the next token
  }
}

// Step 2, the recurrence.  A column j of S (all keys' weights for value element j) never meets
// another column, so a CTA owns some columns of one head of one sequence and walks the tokens in
// order.  A column is cut over LPC adjacent lanes of DPT (32, or 16 where the step has few CTAs
// otherwise) key elements each (d <= DPT LPC), kept in
// registers; the tokens' k, q, v, beta, decay and k . q come through shared memory a tile of tokens at a
// time, the next tile on its way (cp.async) while this one is worked on.
// The read-out after the write, o = S_new^T q, is taken from the state before it:
//     S_new^T q = g S^T q + (k . q) u,
// so that both products with the old state (S^T k and S^T q) run side by side and only one
// multiply-add per element lies between one token's products and the next one's.
// Before they start, the CTAs of a sequence move the convolution state on between them (the raw
// projections of the step's last taps - 1 tokens; step 1 has finished with the old one).
// The slot's S is stored [H][d][dv], so that the lanes of a warp read neighbouring words.
constexpr int DR_THREADS = 128, DR_TILE = 8;

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(float* smem, const float* gmem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int LPC, int DR_DPT>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ prep, const float* __restrict__ bg, const T* __restrict__ proj, long long ld,
                  int conv_col, int taps, float* __restrict__ state, long long state_ld, long long conv_off,
                  float* __restrict__ out, const int* __restrict__ cu_tokens, const int* __restrict__ seq_slots,
                  int H, int G, int d, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int COLS = DR_THREADS / LPC;
    constexpr int DP = DR_DPT * LPC;                      // padded key size
    constexpr int PS = DR_DPT + 4;                        // in shared memory every part starts four banks further on: 16-byte reads without conflicts
    constexpr int DPS = PS * LPC;
    __shared__ __align__(16) float ks[2][DR_TILE][DPS], qs[2][DR_TILE][DPS], vs[2][DR_TILE][COLS], sc[2][DR_TILE][4];
    const int s = blockIdx.z, h = blockIdx.y;
    const int r0 = cu_tokens[s], r1 = cu_tokens[s + 1];
    if (r1 <= r0) return;
    const int slot = seq_slots[s];
    const int C = 2 * G * d + H * dv;
    const int W = 2 * H + G;
    float* slot_state = state + (size_t)slot * state_ld;
    if (taps > 1) {
        float* cs = slot_state + conv_off;
        const int n_new = r1 - r0;
        const int n_ctas = gridDim.x * gridDim.y, mine = blockIdx.y * gridDim.x + blockIdx.x;
        for (int c = mine * DR_THREADS + threadIdx.x; c < C; c += n_ctas * DR_THREADS)
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
    float* sp = slot_state + ((size_t)h * d + part * DR_DPT) * dv + (live ? col : 0);
#pragma unroll
    for (int i = 0; i < DR_DPT; ++i) S[i] = (live && part * DR_DPT + i < d) ? sp[(size_t)i * dv] : 0.f;

    const bool vec = ((d | dv) & 3) == 0 && (((uintptr_t)prep) & 15) == 0;     // rows of prep and the heads in them on 16-byte boundaries
    auto fetch = [&](int b, int t0) {                     // a tile's inputs on their way into buffer b
        const int nt = min(DR_TILE, r1 - t0);
        if (vec) {
            for (int e = threadIdx.x; e < nt * (DP / 4); e += DR_THREADS) {
                const int tt = e / (DP / 4), i = (e - tt * (DP / 4)) * 4;
                const int at = (i / DR_DPT) * PS + i % DR_DPT;
                const float* p = prep + (size_t)(t0 + tt) * C;
                if (i < d) {
                    cp_async16(&ks[b][tt][at], p + (size_t)(G + g) * d + i);
                    cp_async16(&qs[b][tt][at], p + (size_t)g * d + i);
                } else {
                    *reinterpret_cast<float4*>(&ks[b][tt][at]) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(&qs[b][tt][at]) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        } else {
            for (int e = threadIdx.x; e < nt * DP; e += DR_THREADS) {
                const int tt = e / DP, i = e - tt * DP;
                const int at = (i / DR_DPT) * PS + i % DR_DPT;
                const float* p = prep + (size_t)(t0 + tt) * C;
                if (i < d) {
                    cp_async4(&ks[b][tt][at], p + (size_t)(G + g) * d + i);
                    cp_async4(&qs[b][tt][at], p + (size_t)g * d + i);
                } else {
                    ks[b][tt][at] = 0.f;
                    qs[b][tt][at] = 0.f;
                }
            }
        }
        for (int e = threadIdx.x; e < nt * COLS; e += DR_THREADS) {
            const int tt = e / COLS, c = e - tt * COLS;
            const int cc = blockIdx.x * COLS + c;
            if (cc < dv) cp_async4(&vs[b][tt][c], prep + (size_t)(t0 + tt) * C + 2 * G * d + (size_t)h * dv + cc);
            else vs[b][tt][c] = 0.f;
        }
        if (threadIdx.x < nt) {
            const float* p = bg + (size_t)(t0 + threadIdx.x) * W;
            cp_async4(&sc[b][threadIdx.x][0], p + h);
            cp_async4(&sc[b][threadIdx.x][1], p + H + h);
            cp_async4(&sc[b][threadIdx.x][2], p + 2 * H + g);
        }
        cp_async_commit();
    };

    fetch(0, r0);
    int b = 0;
    for (int t0 = r0; t0 < r1; t0 += DR_TILE, b ^= 1) {
        const int nt = min(DR_TILE, r1 - t0);
        if (t0 + DR_TILE < r1) { fetch(b ^ 1, t0 + DR_TILE); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float kk[DR_DPT], qq[DR_DPT];
#pragma unroll
            for (int i = 0; i < DR_DPT; i += 4) {
                *reinterpret_cast<float4*>(&kk[i]) = *reinterpret_cast<const float4*>(&ks[b][tt][part * PS + i]);
                *reinterpret_cast<float4*>(&qq[i]) = *reinterpret_cast<const float4*>(&qs[b][tt][part * PS + i]);
            }
            const float beta = sc[b][tt][0], decay = sc[b][tt][1], kq = sc[b][tt][2];
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
            const float u = beta * (vs[b][tt][col_local] - decay * skt);
#pragma unroll
            for (int i = 0; i < DR_DPT; ++i) S[i] = fmaf(kk[i], u, decay * S[i]);
            if (live && part == 0) out[((size_t)(t0 + tt) * H + h) * dv + col] = fmaf(kq, u, decay * sqt);
        }
        __syncthreads();                                   // the buffer is free for the tile after the next
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DR_DPT; ++i)
            if (part * DR_DPT + i < d) sp[(size_t)i * dv] = S[i];
    }
}

}  // namespace kl

using namespace kl;

// proj: compute dtype [rows, ld]; z, x, g at columns z_col, x_col, g_col (width each); out [rows, width].
// max_new: no sequence brings more rows.  With `chunk_scratch` (float32 [n_seqs * ceil(max_new / MG_CHUNK) * 3 * width]) and a step
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
// state: float32 [slots][state_ld]: S as [H][d][dv] at 0, the convolution state [taps - 1][C] at conv_off.
// prep [rows, C], bg [rows, 2 H + G], out [rows, H * dv]: float32.  max_new: no sequence brings more rows.
KL_API int kl_gated_delta_rule(const void* proj, long long ld, int conv_col, int b_col, int a_col, const float* taps_w, int taps,
                               const float* A_log, const float* dt_bias, float* state, long long state_ld, long long conv_off,
                               float* prep, float* bg, float* out, const int* cu_tokens, const int* seq_slots, int n_seqs,
                               int max_new, int H, int G, int d, int dv, float q_scale, float unit_eps, int dtype,
                               cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return KL_OK;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || taps < 1 || d > 256 || n_seqs > 65535 || G + H > 65535) return KL_ERR_BAD_SIZE;
    const size_t smem = (size_t)(2 * d + 33) * sizeof(float);
    // 32 key elements per lane; 16 (twice the lanes, half the chain per token) where that still leaves SMs without a CTA
    int lpc = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8;
    int dpt = 32;
    const long long ctas32 = (long long)((dv + DR_THREADS / lpc - 1) / (DR_THREADS / lpc)) * H * n_seqs;
    if (d > 16 && ctas32 < 2LL * (sm_count() > 0 ? sm_count() : 1)) {
        dpt = 16;
        lpc = d <= 32 ? 2 : d <= 64 ? 4 : d <= 128 ? 8 : 16;
    }
    const int tpc = max_new >= 256 ? 8 : max_new >= 32 ? 4 : 1;      // tokens a CTA of step 1 walks
    const dim3 grid1((max_new + tpc - 1) / tpc, n_seqs, G + H);
    const dim3 grid2((dv + DR_THREADS / lpc - 1) / (DR_THREADS / lpc), H, n_seqs);
    if (grid2.y > 65535) return KL_ERR_BAD_SIZE;
#define KL_DR(T, L, D) launch_kernel(delta_rule_kernel<T, L, D>, grid2, DR_THREADS, 0, stream, (const float*)prep, (const float*)bg, (const T*)proj, ld, \
                                     conv_col, taps, state, state_ld, conv_off, out, cu_tokens, seq_slots, H, G, d, dv)
#define KL_DELTA(T)                                                                                                          \
    do {                                                                                                                     \
        launch_kernel(delta_prepare_kernel<T>, grid1, DP_THREADS, smem, stream, (const T*)proj, ld, conv_col, b_col, a_col, taps_w, taps, A_log, \
                      dt_bias, (const float*)state, state_ld, conv_off, prep, bg, cu_tokens, seq_slots, H, G, d, dv, q_scale, unit_eps, tpc); \
        KL_LAUNCH_CHECK();                                                                                                   \
        if (dpt == 32) { if (lpc == 1) KL_DR(T, 1, 32); else if (lpc == 2) KL_DR(T, 2, 32); else if (lpc == 4) KL_DR(T, 4, 32); else KL_DR(T, 8, 32); } \
        else { if (lpc == 2) KL_DR(T, 2, 16); else if (lpc == 4) KL_DR(T, 4, 16); else if (lpc == 8) KL_DR(T, 8, 16); else KL_DR(T, 16, 16); } \
    } while (0)
    if (dtype == KL_F32) KL_DELTA(float);
    else if (dtype == KL_BF16) KL_DELTA(bf16);
    else return KL_ERR_BAD_DTYPE;
#undef KL_DELTA
#undef KL_DR
    KL_LAUNCH_CHECK();
    return KL_OK;
}
