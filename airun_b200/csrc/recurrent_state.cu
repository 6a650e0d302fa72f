// Two recurrent mixers whose state is a matrix per head, and what feeds them.
//
// Delta rule with a decay per key channel (per head, key channels d < D, value channels j < Dv, token by token):
//     S[d][j] <- g_t[d] * S[d][j]
//     u[j]     = beta_t * (v_t[j] - sum_d S[d][j] * k_t[d])
//     S[d][j] <- S[d][j] + k_t[d] * u[j]
//     o_t[j]   = sum_d S[d][j] * q_t[d]                      (the read-out sees the token's own write)
// Time mix with a bonus for the current token (value channels j < D as well):
//     o_t[j]   = sum_d r_t[d] * (S[d][j] + u[d] * k_t[d] * v_t[j])
//     S[d][j] <- w_t[d] * S[d][j] + k_t[d] * v_t[j]
// Both run in float32 on a state that lives in the request's slot of a state tensor between steps, [D][Dv] per
// head, so the result at a token depends on the request's tokens up to it and on nothing else: not on how they
// were cut into steps, not on the batch around them.
//
// The delta rule's q, k and v pass a short causal convolution over time per channel and silu, and q and k are
// made unit vectors per head (short_conv_kernel); the last taps - 1 inputs of the convolution are state too.  The
// time mix reads, per projection, x_t + (x_{t-1} - x_t) * mu (token_shift_kernel); x of the last token is state.
#include "common.cuh"

// ------------------------------------------------------------------------------------------ short convolution
// in [T][C] (row stride in_stride) holds the inputs of C channels: first n_unit_heads heads of `unit_dim`
// channels whose outputs are made unit vectors (x / sqrt(sum x^2 + unit_eps)), the first q_heads of them also
// times q_scale; the rest is left as silu gives it.  y[t][c] = silu(sum_j w[c][j] * in[t - (taps-1) + j][c]);
// rows before the request's first row of this step come from tail[slot][taps-1][C] (the inputs that ended the
// step before; zero at the start of a request).  One block per token.
__global__ __launch_bounds__(256) void short_conv_kernel(
    const float* __restrict__ in, long long in_stride, const float* __restrict__ w, int taps,
    const float* __restrict__ state, long long slot_stride, long long tail_off, int max_slots,
    const int32_t* __restrict__ req_of_token, const int32_t* __restrict__ cu_tokens, const int32_t* __restrict__ state_slots,
    int num_reqs, float* __restrict__ out, int C, int n_unit_heads, int q_heads, int unit_dim, float unit_eps,
    float q_scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_y[];                 // [C]
    const int t = blockIdx.x;
    const int req = req_of_token[t];
    if (req < 0) return;
    if (req >= num_reqs) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ); return; }
    const int slot = state_slots[req];
    if (slot < 0 || slot >= max_slots) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ); return; }
    const int i = t - cu_tokens[req];              // place of the token within its request's rows of this step
    const float* tail = state + (size_t)slot * slot_stride + tail_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int src = i - (taps - 1) + j;
            const float xv = src >= 0 ? in[(size_t)(t - (taps - 1) + j) * in_stride + c] : tail[(size_t)(i + j) * C + c];
            acc = fmaf(w[(size_t)c * taps + j], xv, acc);
        }
        s_y[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int h = warp; h < n_unit_heads; h += nwarp) {
        float ss = 0.0f;
        for (int d = lane; d < unit_dim; d += 32) { const float v = s_y[h * unit_dim + d]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float inv = (1.0f / sqrtf(ss + unit_eps)) * (h < q_heads ? q_scale : 1.0f);
        for (int d = lane; d < unit_dim; d += 32) out[(size_t)t * C + h * unit_dim + d] = s_y[h * unit_dim + d] * inv;
    }
    for (int c = n_unit_heads * unit_dim + threadIdx.x; c < C; c += blockDim.x) out[(size_t)t * C + c] = s_y[c];
}

AIRUN_EXPORT int airun_short_conv(const float* in, long long in_stride, const float* w, int taps, const float* state,
                                  long long slot_stride, long long tail_off, int max_slots, const int32_t* req_of_token,
                                  const int32_t* cu_tokens, const int32_t* state_slots, int num_reqs, float* out, int T, int C,
                                  int n_unit_heads, int q_heads, int unit_dim, float unit_eps, float q_scale, int* err,
                                  cudaStream_t stream) {
    if (T < 0 || C <= 0 || taps <= 0 || taps > 64 || in_stride < C || !state || !err || n_unit_heads < 0 || unit_dim <= 0 ||
        (long long)n_unit_heads * unit_dim > C || C > 48 * 1024 / 4)
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    airun_launch(short_conv_kernel, dim3(T), dim3(256), (size_t)C * sizeof(float), stream, in, in_stride, w, taps, state, slot_stride,
                 tail_off, max_slots, req_of_token, cu_tokens, state_slots, num_reqs, out, C, n_unit_heads, q_heads, unit_dim,
                 unit_eps, q_scale, err);
    return airun_launch_status();
}

// ------------------------------------------------------------------------------------------ token shift
// out[s][t][c] = x[t][c] + (prev[c] - x[t][c]) * mu[s][c] for s < n_mix, in the type of `out`; prev is x[t-1], or,
// for the first row a request brings in this step, the row its state keeps (zero at the start of a request).
template <typename TOut>
__global__ __launch_bounds__(256) void token_shift_kernel(
    const float* __restrict__ x, const float* __restrict__ mu, int n_mix, const float* __restrict__ state,
    long long slot_stride, long long prev_off, int max_slots, const int32_t* __restrict__ req_of_token,
    const int32_t* __restrict__ cu_tokens, const int32_t* __restrict__ state_slots, int num_reqs, TOut* __restrict__ out,
    int T, int W, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int req = req_of_token[t];
    if (req < 0) return;
    if (req >= num_reqs) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ); return; }
    const int slot = state_slots[req];
    if (slot < 0 || slot >= max_slots) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ); return; }
    const float* prev = t > cu_tokens[req] ? x + (size_t)(t - 1) * W : state + (size_t)slot * slot_stride + prev_off;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float xv = x[(size_t)t * W + c], d = prev[c] - xv;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * T + t) * W + c] = from_f32<TOut>(fmaf(d, mu[(size_t)s * W + c], xv));
    }
}

AIRUN_EXPORT int airun_token_shift(const float* x, const float* mu, int n_mix, const float* state, long long slot_stride,
                                   long long prev_off, int max_slots, const int32_t* req_of_token, const int32_t* cu_tokens,
                                   const int32_t* state_slots, int num_reqs, void* out, int out_dtype, int T, int W, int* err,
                                   cudaStream_t stream) {
    if (T < 0 || W <= 0 || n_mix <= 0 || !state || !err) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    if (out_dtype == AIRUN_DT_F32)
        airun_launch(token_shift_kernel<float>, dim3(T), dim3(256), 0, stream, x, mu, n_mix, state, slot_stride, prev_off, max_slots,
                     req_of_token, cu_tokens, state_slots, num_reqs, (float*)out, T, W, err);
    else if (out_dtype == AIRUN_DT_BF16)
        airun_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, x, mu, n_mix, state, slot_stride, prev_off,
                     max_slots, req_of_token, cu_tokens, state_slots, num_reqs, (__nv_bfloat16*)out, T, W, err);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// ------------------------------------------------------------------------------------------ the recurrences
// One block per (request, head, 128 / DG value columns), 128 threads.  A value column is shared by DG = 4 or 8
// neighbouring lanes, each of which keeps NS key channels of the column's state in registers for the whole step: the
// sums over key channels are NS multiply-adds in a thread and two or three shuffles, and nothing but the state chains
// one token to the next.  The key channels of a lane are every DG-th group of four, so the lanes of a column read
// neighbouring float4 of the token's q, k and decay from shared memory.  (Eight lanes a column from 33 key channels
// on: what bounds a prompt is the chain of its tokens, and a warp's instructions per token halve.)  Tokens are staged through shared memory
// a few at a time by asynchronous copies into one of two stages.  The block (request, 0, 0) also moves the request's small state on: the last inputs of the
// short convolution (delta rule) or the last token's x (time mix).
#define RS_TT 16
#define RS_DELTA 0
#define RS_WKV 1

struct RecurrentArgs {
    const float* q; const float* k; const float* v; const float* g;     // delta: q, k, v, decay; time mix: r, k, v, decay
    long long q_stride, k_stride, v_stride, g_stride;                    // row strides in elements
    const float* beta; long long beta_stride;                            // delta: [T][heads], before its sigmoid
    const float* bonus;                                                  // time mix: [heads][D]
    float* state; long long slot_stride; int max_slots;
    const int32_t* cu_tokens; const int32_t* state_slots;
    float* out;                                                          // [T][heads * Dv]
    int heads, kv_rep, D, Dv;                                            // head h reads q/k head h / kv_rep
    // the small state moved on by block (r, 0, 0)
    const float* tail_src; long long tail_src_stride; long long tail_off; int tail_rows, tail_width;
    int* err;
};

__device__ __forceinline__ void rs_cp4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void rs_cp16(float* smem, const float* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

template <int MODE, int NS, int DG>
__global__ __launch_bounds__(128) void recurrent_state_kernel(RecurrentArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int DP = NS * DG;
    constexpr int COLS = 128 / DG;               // value columns of a block: 32 / DG a warp
    constexpr int TT = DP >= 256 ? 4 : DP >= 128 ? 8 : RS_TT;     // tokens of a stage (static shared memory stays under 48 KB)
    // two stages: the next tokens arrive by asynchronous copies while these are used
    __shared__ __align__(16) float s_q[2][TT][DP], s_k[2][TT][DP], s_g[2][TT][DP], s_v[2][TT][COLS];
    __shared__ float s_b[2][TT];
    const int r = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * COLS;
    const int t0 = a.cu_tokens[r], n = a.cu_tokens[r + 1] - t0;
    if (n <= 0) return;
    const int slot = a.state_slots[r];
    if (slot < 0 || slot >= a.max_slots) {
        if (threadIdx.x == 0) atomicOr(a.err, AIRUN_DEV_BAD_REQ);
        return;
    }
    const int D = a.D, Dv = a.Dv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dg = lane & (DG - 1), cl = warp * (32 / DG) + lane / DG, col = col0 + cl;
    const bool col_ok = col < Dv;
    const int qk_head = head / a.kv_rep;
    const int ncol = min(COLS, Dv - col0);
    // the padding beyond D and Dv is zero in both stages and is never copied into (nothing to do when there is none)
    if (D < DP || ncol < COLS) {
        for (int e = threadIdx.x; e < 2 * TT * DP; e += 128) { (&s_q[0][0][0])[e] = 0.0f; (&s_k[0][0][0])[e] = 0.0f; (&s_g[0][0][0])[e] = 0.0f; }
        for (int e = threadIdx.x; e < 2 * TT * COLS; e += 128) (&s_v[0][0][0])[e] = 0.0f;
        __syncthreads();
    }
    const float* qh = a.q + (size_t)qk_head * D;
    const float* kh = a.k + (size_t)qk_head * D;
    const float* gh = a.g + (size_t)head * D;
    const float* vh = a.v + (size_t)head * Dv + col0;
    const bool vec = (D % 4 == 0) && ((a.q_stride | a.k_stride | a.g_stride) % 4 == 0) &&
                     ((((uintptr_t)qh | (uintptr_t)kh | (uintptr_t)gh) & 15) == 0);
    const bool vvec = (ncol % 4 == 0) && (a.v_stride % 4 == 0) && (((uintptr_t)vh & 15) == 0);
    auto stage = [&](int base, int buf) {
        const int nt = min(TT, n - base);
        if (vec) {
            const int per = D / 4;
            for (int e = threadIdx.x; e < nt * per; e += 128) {
                const int tt = e / per, d = (e - tt * per) * 4;
                const size_t row = (size_t)(t0 + base + tt);
                rs_cp16(&s_q[buf][tt][d], qh + row * a.q_stride + d);
                rs_cp16(&s_k[buf][tt][d], kh + row * a.k_stride + d);
                rs_cp16(&s_g[buf][tt][d], gh + row * a.g_stride + d);
            }
        } else {
            for (int e = threadIdx.x; e < nt * D; e += 128) {
                const int tt = e / D, d = e - tt * D;
                const size_t row = (size_t)(t0 + base + tt);
                rs_cp4(&s_q[buf][tt][d], qh + row * a.q_stride + d);
                rs_cp4(&s_k[buf][tt][d], kh + row * a.k_stride + d);
                rs_cp4(&s_g[buf][tt][d], gh + row * a.g_stride + d);
            }
        }
        if (vvec) {
            const int per = ncol / 4;
            for (int e = threadIdx.x; e < nt * per; e += 128) {
                const int tt = e / per, c = (e - tt * per) * 4;
                rs_cp16(&s_v[buf][tt][c], vh + (size_t)(t0 + base + tt) * a.v_stride + c);
            }
        } else {
            for (int e = threadIdx.x; e < nt * ncol; e += 128) {
                const int tt = e / ncol, c = e - tt * ncol;
                rs_cp4(&s_v[buf][tt][c], vh + (size_t)(t0 + base + tt) * a.v_stride + c);
            }
        }
        if (MODE == RS_DELTA && threadIdx.x < nt)
            rs_cp4(&s_b[buf][threadIdx.x], a.beta + (size_t)(t0 + base + threadIdx.x) * a.beta_stride + head);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    float* sbase = a.state + (size_t)slot * a.slot_stride + (size_t)head * D * Dv + (col_ok ? col : 0);
    // channel of register i: group of four (i / 4) * DG + dg, element i % 4
    float S[NS], bonus[MODE == RS_WKV ? NS : 1];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int d = ((i >> 2) * DG + dg) * 4 + (i & 3);
        S[i] = (col_ok && d < D) ? sbase[(size_t)d * Dv] : 0.0f;
        if (MODE == RS_WKV) bonus[i] = d < D ? a.bonus[(size_t)head * D + d] : 0.0f;
    }
    float* orow = a.out + (size_t)t0 * ((size_t)a.heads * Dv) + (size_t)head * Dv + col;
    int it = 0;
    for (int base = 0; base < n; base += TT, ++it) {
        const int buf = it & 1, nt = min(TT, n - base);
        if (base + TT < n) {
            stage(base + TT, buf ^ 1);          // that stage was last read before the barrier that ended the iteration before
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = s_v[buf][tt][cl];
            float o;
            if (MODE == RS_DELTA) {
                // beta arrives as the projection's output: the gate is its sigmoid
                const float beta = 1.0f / (1.0f + expf(-s_b[buf][tt]));
                float pred[2] = {0.0f, 0.0f}, oq[2] = {0.0f, 0.0f}, kq[2] = {0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < NS / 4; ++i4) {
                    const int d = (i4 * DG + dg) * 4;
                    const float4 g4 = *reinterpret_cast<const float4*>(&s_g[buf][tt][d]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[buf][tt][d]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&s_q[buf][tt][d]);
                    const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float sd = gg[e] * S[4 * i4 + e];
                        S[4 * i4 + e] = sd;
                        pred[e & 1] = fmaf(sd, kk[e], pred[e & 1]);
                        oq[e & 1] = fmaf(sd, qq[e], oq[e & 1]);
                        kq[e & 1] = fmaf(kk[e], qq[e], kq[e & 1]);
                    }
                }
                float p = pred[0] + pred[1], oqs = oq[0] + oq[1], kqs = kq[0] + kq[1];
#pragma unroll
                for (int off = 1; off < DG; off <<= 1) {
                    p += __shfl_xor_sync(0xffffffffu, p, off);
                    oqs += __shfl_xor_sync(0xffffffffu, oqs, off);
                    kqs += __shfl_xor_sync(0xffffffffu, kqs, off);
                }
                const float u = beta * (vj - p);
#pragma unroll
                for (int i4 = 0; i4 < NS / 4; ++i4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[buf][tt][(i4 * DG + dg) * 4]);
                    S[4 * i4 + 0] = fmaf(k4.x, u, S[4 * i4 + 0]);
                    S[4 * i4 + 1] = fmaf(k4.y, u, S[4 * i4 + 1]);
                    S[4 * i4 + 2] = fmaf(k4.z, u, S[4 * i4 + 2]);
                    S[4 * i4 + 3] = fmaf(k4.w, u, S[4 * i4 + 3]);
                }
                o = fmaf(u, kqs, oqs);
            } else {
                float ro[2] = {0.0f, 0.0f}, ruk[2] = {0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < NS / 4; ++i4) {
                    const int d = (i4 * DG + dg) * 4;
                    const float4 g4 = *reinterpret_cast<const float4*>(&s_g[buf][tt][d]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[buf][tt][d]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&s_q[buf][tt][d]);
                    const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        ro[e & 1] = fmaf(qq[e], S[4 * i4 + e], ro[e & 1]);
                        ruk[e & 1] = fmaf(qq[e] * bonus[4 * i4 + e], kk[e], ruk[e & 1]);
                        S[4 * i4 + e] = fmaf(gg[e], S[4 * i4 + e], kk[e] * vj);
                    }
                }
                float rs = ro[0] + ro[1], us = ruk[0] + ruk[1];
#pragma unroll
                for (int off = 1; off < DG; off <<= 1) {
                    rs += __shfl_xor_sync(0xffffffffu, rs, off);
                    us += __shfl_xor_sync(0xffffffffu, us, off);
                }
                o = fmaf(vj, us, rs);
            }
            if (dg == 0 && col_ok) orow[(size_t)(base + tt) * ((size_t)a.heads * Dv)] = o;
        }
        __syncthreads();
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int d = ((i >> 2) * DG + dg) * 4 + (i & 3);
            if (d < D) sbase[(size_t)d * Dv] = S[i];
        }
    }
    // the small state: its last `tail_rows` rows become the last rows of (what it held, then this step's rows)
    if (blockIdx.y == 0 && blockIdx.z == 0 && a.tail_rows > 0) {
        float* tail = a.state + (size_t)slot * a.slot_stride + a.tail_off;
        const int R = a.tail_rows, Wd = a.tail_width;
        for (int c = threadIdx.x; c < Wd; c += 128) {
            for (int s = 0; s < R; ++s) {            // row s comes from a later row: ascending s never reads what it wrote
                const int src = s + n;
                tail[(size_t)s * Wd + c] = src < R ? tail[(size_t)src * Wd + c]
                                                   : a.tail_src[(size_t)(t0 + src - R) * a.tail_src_stride + c];
            }
        }
    }
}

AIRUN_EXPORT int airun_recurrent_state(int mode, const float* q, const float* k, const float* v, const float* g,
                                       long long q_stride, long long k_stride, long long v_stride, long long g_stride,
                                       const float* beta, long long beta_stride, const float* bonus, float* state,
                                       long long slot_stride, int max_slots, const int32_t* cu_tokens, const int32_t* state_slots,
                                       int num_reqs, float* out, int heads, int kv_rep, int D, int Dv, const float* tail_src,
                                       long long tail_src_stride, long long tail_off, int tail_rows, int tail_width,
                                       int long_chains, int* err, cudaStream_t stream) {
    if (num_reqs < 0 || heads <= 0 || heads > 65535 || kv_rep <= 0 || heads % kv_rep || D <= 0 || D > 256 || Dv <= 0 || !state ||
        !cu_tokens || !state_slots || !err || !q || !k || !v || !g || !out || slot_stride < (long long)heads * D * Dv)
        return AIRUN_ERR_ARG;
    if (mode == RS_DELTA ? !beta : !bonus) return AIRUN_ERR_ARG;
    if (tail_rows < 0 || (tail_rows > 0 && (!tail_src || tail_width <= 0))) return AIRUN_ERR_ARG;
    if (num_reqs == 0) return AIRUN_OK;
    // lanes that share a value column: 8 where requests bring many tokens (the chain of a prompt's tokens bounds the
    // step, and a warp's instructions per token halve), 4 where most bring one (the state is read and written once, in
    // wider pieces)
    const int dg = (D <= 32 || !long_chains) ? 4 : 8;
    const int tiles = ceil_div_i(Dv, 128 / dg);
    if (tiles > 65535) return AIRUN_ERR_ARG;
    RecurrentArgs a = {q, k, v, g, q_stride, k_stride, v_stride, g_stride, beta, beta_stride, bonus, state, slot_stride, max_slots,
                       cu_tokens, state_slots, out, heads, kv_rep, D, Dv, tail_src, tail_src_stride, tail_off, tail_rows,
                       tail_width, err};
    dim3 grid(num_reqs, heads, tiles);
#define RS_LAUNCH(NS, DG) \
    do { if (mode == RS_DELTA) airun_launch(recurrent_state_kernel<RS_DELTA, NS, DG>, grid, dim3(128), 0, stream, a); \
         else airun_launch(recurrent_state_kernel<RS_WKV, NS, DG>, grid, dim3(128), 0, stream, a); } while (0)
    if (D <= 16) RS_LAUNCH(4, 4);
    else if (D <= 32) RS_LAUNCH(8, 4);
    else if (D <= 64) { if (dg == 8) RS_LAUNCH(8, 8); else RS_LAUNCH(16, 4); }
    else if (D <= 128) { if (dg == 8) RS_LAUNCH(16, 8); else RS_LAUNCH(32, 4); }
    else { if (dg == 8) RS_LAUNCH(32, 8); else RS_LAUNCH(64, 4); }
#undef RS_LAUNCH
    return airun_launch_status();
}
