// Differential attention of prompt portions and of single decoded tokens on the tensor cores (mma.sync m16n8k16,
// bfloat16 operands, float32 accumulation).  The formulas and the page layout are those of
// diff_attention.cu, its plain twin; this file only computes them tile by tile.
//
// One CTA (4 warps) takes up to 64 consecutive tokens of one request and one query head; a warp owns 16 of
// them.  The CTA finds its tile by walking the requests' token counts (cu_tokens), so the launch needs
// nothing from the host but an upper bound of the tile count: ceil(T / 64) + requests.  The keys the tile
// can see, from the start of the chunk (or window) of its first token to its last token, are walked in
// tiles of 64: K and V rows are staged in shared memory as bfloat16 (16-byte copies when D and Dv are multiples
// of 8; V reaches the second product transposed by ldmatrix), and for each of the two
// maps in turn the warp forms S = Q_m K_m^T, applies scale, soft cap and mask in float32, updates the
// running maximum and sum of its rows (online softmax) and adds P_m V to the map's accumulator.  At the
// end o = a_1 - lambda * a_2 is divided by its root mean square over the head and scaled.
//
// D and Dv are padded to the template sizes DP and DVP with zeros in shared memory, so any D, Dv up to 128
// run; which (DP, DVP) pair a call uses is chosen by the launcher.  A token's result does not depend on
// the other rows of its tile or on the batch: every row keeps its own maximum and sum, and keys are added
// in the same order (tiles counted from the first key ITS tile can see; rows of one tile share that start).
#include "common.cuh"

#define DAM_ROWS 64
#define DAM_KEYS 64
#define DAM_PAD 8

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct DamParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    long long out_stride;
    const __nv_bfloat16* pool;
    const int32_t* block_table;
    int max_blocks;
    const int32_t* cu_tokens;
    const int32_t* context_lens;
    int num_reqs, num_pages, page_size, nh, nkv, D, Dv;
    float scale, cap, lambda, eps, out_scale;
    int chunk, window;
    int skip_single;              // requests that bring ONE token are left to the kernel for single tokens
    int* err;
};

template <int DP, int DVP>
__global__ __launch_bounds__(128) void diff_attention_mma_kernel(const DamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = 2 * DP + DAM_PAD;          // row stride of Qs and Ks in elements
    constexpr int VS = DVP + DAM_PAD;             // row stride of Vs
    extern __shared__ __align__(16) unsigned char dam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(dam_smem);            // [64][QS]
    __nv_bfloat16* Ks0 = Qs + DAM_ROWS * QS;                                   // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * DAM_KEYS * QS;                              // [2][64][VS]
    // ---- which tile
    // (tiles later in a request see more keys: the grid is walked from its end so that they start first)
    int b = gridDim.y - 1 - blockIdx.y, req = -1, first = 0, n = 0, ctx_len = 0;
    for (int r = 0; r < p.num_reqs; ++r) {
        const int t0 = p.cu_tokens[r], nr = p.cu_tokens[r + 1] - t0;
        if (nr <= 0 || (p.skip_single && nr == 1)) continue;
        const int tiles = (nr + DAM_ROWS - 1) / DAM_ROWS;
        if (b < tiles) { req = r; first = t0 + b * DAM_ROWS; n = min(DAM_ROWS, nr - b * DAM_ROWS); ctx_len = p.context_lens[r];
                         ctx_len = ctx_len - nr + b * DAM_ROWS; break; }      // position of the tile's first token
        b -= tiles;
    }
    if (req < 0) return;
    const int p0 = ctx_len;
    const int head = blockIdx.x, kvh = head / (p.nh / p.nkv);
    const int D = p.D, Dv = p.Dv, kd = 2 * D;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // ---- shared memory starts as zeros (the padding beyond D and Dv stays so), then the Q tile
    const bool vec = (D % 8 == 0) && (Dv % 8 == 0);
    {
        constexpr int WORDS16 = (3 * DAM_ROWS * QS + 2 * DAM_KEYS * VS) / 8;
        uint4* z = reinterpret_cast<uint4*>(dam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    if (vec) {
        const int per = kd / 8;
        for (int e = tid; e < n * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8, m = c / D, d = c - m * D;
            cp_async16(Qs + row * QS + m * DP + d, p.q + ((size_t)(first + row) * p.nh + head) * kd + c);
        }
    } else {
        for (int e = tid; e < n * kd; e += 128) {
            const int row = e / kd, c = e - row * kd, m = c / D, d = c - m * D;
            Qs[row * QS + m * DP + d] = p.q[((size_t)(first + row) * p.nh + head) * kd + c];
        }
    }
    int lo = p.chunk > 0 ? (p0 / p.chunk) * p.chunk : 0;
    if (p.window > 0) lo = max(lo, p0 - p.window + 1);
    const int hi = p0 + n - 1;
    // rows of this thread: r0 = warp * 16 + g and r0 + 8
    int pos[2], vis_lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + 8 * h;
        pos[h] = row < n ? p0 + row : -1;
        int s = p.chunk > 0 && pos[h] >= 0 ? (pos[h] / p.chunk) * p.chunk : 0;
        if (p.window > 0) s = max(s, pos[h] - p.window + 1);
        vis_lo[h] = s;
    }
    float O[2][DVP / 8][4];
    float mx[2][2], sm[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int h = 0; h < 2; ++h) { mx[m][h] = -INFINITY; sm[m][h] = 0.0f; }
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) O[m][i][j] = 0.0f;
    }
    const size_t page_elems = (size_t)p.nkv * p.page_size * (kd + Dv);
    const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
    const float inv_cap = p.cap > 0.0f ? 1.0f / p.cap : 0.0f;
    bool bad = false;
    // K and V rows of up to 64 keys from kbase on into stage `buf` (rows beyond the last key keep what they held:
    // they are masked).  With 16-byte rows the copies are asynchronous and the next tile is on its way while
    // this one is used.
    // when the 16-byte pieces of a key's rows divide the CTA's threads evenly and pages are a power of two, each thread
    // owns one piece (reg_*: where it lies in the page and in shared memory) for every key it copies
    const int reg_lp = max(1, kd / 8 + Dv / 8);
    const bool regular = vec && reg_lp <= 128 && 128 % reg_lp == 0 && (p.page_size & (p.page_size - 1)) == 0;
    const int ps_shift = __ffs(p.page_size) - 1;
    const int reg_u = tid % reg_lp, reg_key0 = tid / reg_lp, reg_step = 128 / reg_lp;
    const bool reg_is_k = reg_u < kd / 8;
    const int reg_c = reg_is_k ? reg_u * 8 : (reg_u - kd / 8) * 8;
    const int reg_dst = reg_is_k ? (reg_c / D) * DP + reg_c % D : reg_c;
    const int reg_stride = reg_is_k ? QS : VS, reg_row = reg_is_k ? kd : Dv;
    const size_t reg_src = reg_is_k ? (size_t)kvh * p.page_size * kd + reg_c
                                    : (size_t)p.nkv * p.page_size * kd + (size_t)kvh * p.page_size * Dv + reg_c;
    auto load_tile = [&](int kbase, int buf) {
        __nv_bfloat16* Ks = Ks0 + buf * DAM_KEYS * QS;
        __nv_bfloat16* Vs = Vs0 + buf * DAM_KEYS * VS;
        const int nk = min(DAM_KEYS, hi - kbase + 1);
        if (regular) {
            // a thread keeps its 16-byte column of the key (or value) row and walks the keys: nothing but the page
            // lookup is worked out per copy
            __nv_bfloat16* dst = (reg_is_k ? Ks : Vs) + reg_dst;
            for (int key = reg_key0; key < nk; key += reg_step) {
                const int j = kbase + key, blk = j >> ps_shift;
                const int page = blk < p.max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= p.num_pages) { bad = true; continue; }
                cp_async16(dst + key * reg_stride, p.pool + (size_t)page * page_elems + reg_src + (size_t)(j & (p.page_size - 1)) * reg_row);
            }
            cp_async_commit();
            return;
        }
        const int perk = vec ? kd / 8 : kd, perv = vec ? Dv / 8 : Dv;
        for (int e = tid; e < nk * (perk + perv); e += 128) {
            const int key = e / (perk + perv), u = e - key * (perk + perv);
            const int j = kbase + key, blk = j / p.page_size;
            const int page = blk < p.max_blocks ? bt[blk] : -1;
            if (page < 0 || page >= p.num_pages) { bad = true; continue; }
            const __nv_bfloat16* pk = p.pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * kd;
            const __nv_bfloat16* pv = p.pool + (size_t)page * page_elems + (size_t)p.nkv * p.page_size * kd +
                                      ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * Dv;
            if (vec) {
                if (u < perk) {
                    const int c = u * 8, m = c / D, d = c - m * D;
                    cp_async16(Ks + key * QS + m * DP + d, pk + c);
                } else {
                    const int c = (u - perk) * 8;
                    cp_async16(Vs + key * VS + c, pv + c);
                }
            } else if (u < perk) {
                const int m = u / D, d = u - m * D;
                Ks[key * QS + m * DP + d] = pk[u];
            } else {
                Vs[key * VS + (u - perk)] = pv[u - perk];
            }
        }
        cp_async_commit();
    };
    load_tile(lo, 0);
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += DAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * DAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * DAM_KEYS * VS;
        if (kbase + DAM_KEYS <= hi) {
            load_tile(kbase + DAM_KEYS, buf ^ 1);          // its stage was last read before the barrier that ended the tile before
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp * 16 < n)                                 // a warp without rows only helps to load
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float S[DAM_KEYS / 8][4];
#pragma unroll
            for (int i = 0; i < DAM_KEYS / 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) S[i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DP / 16; ++ks) {
                uint32_t a[4];
                const __nv_bfloat16* qa = Qs + (warp * 16 + g) * QS + m * DP + ks * 16 + 2 * t;
                a[0] = *reinterpret_cast<const uint32_t*>(qa);
                a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS);
                a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + 8);
#pragma unroll
                for (int nt = 0; nt < DAM_KEYS / 8; ++nt) {
                    const __nv_bfloat16* kb = Ks + (nt * 8 + g) * QS + m * DP + ks * 16 + 2 * t;
                    mma_bf16(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
            // ---- scale, cap, mask, running maximum.  The cap c * tanh(x / c) = c - 2c / (exp(2x / c) + 1) with the
            // scale and log2(e) folded into one factor; the mask only where a key of the tile can be hidden from a
            // row of this warp; the exponentials in base 2 with the maximum folded into one multiply-add.
            const float LOG2E = 1.4426950408889634f;
            const float cap_in = 2.0f * p.scale * inv_cap * LOG2E, cap2 = -2.0f * p.cap;
            const int row_lo = p0 + warp * 16, row_hi = min(p0 + warp * 16 + 15, hi);
            int need_lo = lo;                               // the latest first-visible key among the warp's rows
            if (p.chunk > 0) need_lo = max(need_lo, (row_hi / p.chunk) * p.chunk);
            if (p.window > 0) need_lo = max(need_lo, row_hi - p.window + 1);
            const bool masked = kbase + DAM_KEYS - 1 > row_lo || kbase < need_lo || warp * 16 + 15 >= n;
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < DAM_KEYS / 8; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    float s;
                    if (p.cap > 0.0f) s = fmaf(cap2, __fdividef(1.0f, exp2f(S[nt][j] * cap_in) + 1.0f), p.cap);
                    else s = S[nt][j] * p.scale;
                    if (masked) {
                        const int key = kbase + nt * 8 + 2 * t + (j & 1);
                        s = (key <= pos[h] && key >= vis_lo[h]) ? s : -INFINITY;
                    }
                    S[nt][j] = s;
                    tmax[h] = fmaxf(tmax[h], s);
                }
            float corr[2], mnew[2], mneg[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                mnew[h] = fmaxf(mx[m][h], tmax[h]);
                corr[h] = mnew[h] == -INFINITY ? 1.0f : exp2f((mx[m][h] - mnew[h]) * LOG2E);      // 0 on the first keys
                mx[m][h] = mnew[h];
                mneg[h] = mnew[h] == -INFINITY ? 0.0f : -mnew[h] * LOG2E;      // a row that sees nothing yet: exp2(-inf) = 0
            }
            float tsum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int nt = 0; nt < DAM_KEYS / 8; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    const float pr = exp2f(fmaf(S[nt][j], LOG2E, mneg[h]));
                    S[nt][j] = pr;
                    tsum[h] += pr;
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 1);
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 2);
                sm[m][h] = sm[m][h] * corr[h] + tsum[h];
            }
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                O[m][i][0] *= corr[0]; O[m][i][1] *= corr[0];
                O[m][i][2] *= corr[1]; O[m][i][3] *= corr[1];
            }
            // ---- O_m += P V
#pragma unroll
            for (int kk = 0; kk < DAM_KEYS / 16; ++kk) {
                uint32_t a[4];
                a[0] = pack_bf16(S[2 * kk][0], S[2 * kk][1]);
                a[1] = pack_bf16(S[2 * kk][2], S[2 * kk][3]);
                a[2] = pack_bf16(S[2 * kk + 1][0], S[2 * kk + 1][1]);
                a[3] = pack_bf16(S[2 * kk + 1][2], S[2 * kk + 1][3]);
#pragma unroll
                for (int nv = 0; nv < DVP / 8; ++nv) {
                    // keys kk*16 .. +15 (rows of Vs) x columns nv*8 .. +7, transposed on the way
                    uint32_t b0, b1;
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + (lane & 15)) * VS + nv * 8);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                    mma_bf16(O[m][nv], a, b0, b1);
                }
            }
        }
        __syncthreads();                                   // this stage may be written again
    }
    if (bad && lane == 0) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);
    if (warp * 16 >= n) return;
    // ---- o = a_1 - lambda * a_2, o / rms(o) * out_scale
    float inv[2][2], ss[2] = {0.0f, 0.0f};
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) inv[m][h] = sm[m][h] > 0.0f ? 1.0f / sm[m][h] : 0.0f;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int h = j >> 1;
            const float o = O[0][i][j] * inv[0][h] - p.lambda * (O[1][i][j] * inv[1][h]);
            O[0][i][j] = o;
            ss[h] = fmaf(o, o, ss[h]);          // padded columns hold zeros
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
        ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
        const int row = warp * 16 + g + 8 * h;
        if (row >= n) continue;
        const float nrm = p.out_scale / sqrtf(ss[h] / (float)Dv + p.eps);
        __nv_bfloat16* dst = p.out + (size_t)(first + row) * p.out_stride + (size_t)head * Dv;
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i) {
            const int c = i * 8 + 2 * t;
            if (c < Dv) dst[c] = __float2bfloat16_rn(O[0][i][2 * h] * nrm);
            if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[0][i][2 * h + 1] * nrm);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Single decoded tokens on the tensor cores.  One CTA (4 warps) per (request that brings ONE token, KV head): the
// rows of the products are the G query heads of the group (up to 16), so every key and value row that is read
// serves all of them and both maps.  The visible keys are walked in tiles of 64 through the same two asynchronous
// stages as above; inside a tile warp w takes keys 16w .. 16w+15 (two score tiles and one step of the second
// product per map), with its own running maximum, sum and accumulators; at the end the four warps' results are
// merged through shared memory in warp order, the maps are combined, the heads normed and written.
template <int DP, int DVP>
__global__ __launch_bounds__(128) void diff_attention_group_kernel(const DamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = 2 * DP + DAM_PAD, VS = DVP + DAM_PAD;
    constexpr int PER = 2 * (DVP / 8 * 4 + 4) + 1;          // floats a thread hands to the merge (odd: no bank conflicts)
    extern __shared__ __align__(16) unsigned char dam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(dam_smem);            // [16][QS]
    __nv_bfloat16* Ks0 = Qs + 16 * QS;                                         // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * DAM_KEYS * QS;                              // [2][64][VS]
    const int r = blockIdx.y, kvh = blockIdx.x;
    const int tok = p.cu_tokens[r];
    if (p.cu_tokens[r + 1] - tok != 1) return;
    const int hi = p.context_lens[r] - 1;                  // the token's position: the last key it sees
    const int D = p.D, Dv = p.Dv, kd = 2 * D, G = p.nh / p.nkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const bool vec = (D % 8 == 0) && (Dv % 8 == 0);
    {
        constexpr int WORDS16 = ((16 + 2 * DAM_KEYS) * QS + 2 * DAM_KEYS * VS) / 8;
        uint4* z = reinterpret_cast<uint4*>(dam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    if (vec) {
        const int per = kd / 8;
        for (int e = tid; e < G * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8, m = c / D, d = c - m * D;
            cp_async16(Qs + row * QS + m * DP + d, p.q + ((size_t)tok * p.nh + kvh * G + row) * kd + c);
        }
    } else {
        for (int e = tid; e < G * kd; e += 128) {
            const int row = e / kd, c = e - row * kd, m = c / D, d = c - m * D;
            Qs[row * QS + m * DP + d] = p.q[((size_t)tok * p.nh + kvh * G + row) * kd + c];
        }
    }
    int lo = p.chunk > 0 ? (hi / p.chunk) * p.chunk : 0;
    if (p.window > 0) lo = max(lo, hi - p.window + 1);
    const bool row_on[2] = {g < G, g + 8 < G};
    float O[2][DVP / 8][4], mx[2][2], sm[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int h = 0; h < 2; ++h) { mx[m][h] = -INFINITY; sm[m][h] = 0.0f; }
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) O[m][i][j] = 0.0f;
    }
    const size_t page_elems = (size_t)p.nkv * p.page_size * (kd + Dv);
    const int32_t* bt = p.block_table + (size_t)r * p.max_blocks;
    const float inv_cap = p.cap > 0.0f ? 1.0f / p.cap : 0.0f;
    const float LOG2E = 1.4426950408889634f;
    const float cap_in = 2.0f * p.scale * inv_cap * LOG2E, cap2 = -2.0f * p.cap;
    bool bad = false;
    // when the 16-byte pieces of a key's rows divide the CTA's threads evenly and pages are a power of two, each thread
    // owns one piece (reg_*: where it lies in the page and in shared memory) for every key it copies
    const int reg_lp = max(1, kd / 8 + Dv / 8);
    const bool regular = vec && reg_lp <= 128 && 128 % reg_lp == 0 && (p.page_size & (p.page_size - 1)) == 0;
    const int ps_shift = __ffs(p.page_size) - 1;
    const int reg_u = tid % reg_lp, reg_key0 = tid / reg_lp, reg_step = 128 / reg_lp;
    const bool reg_is_k = reg_u < kd / 8;
    const int reg_c = reg_is_k ? reg_u * 8 : (reg_u - kd / 8) * 8;
    const int reg_dst = reg_is_k ? (reg_c / D) * DP + reg_c % D : reg_c;
    const int reg_stride = reg_is_k ? QS : VS, reg_row = reg_is_k ? kd : Dv;
    const size_t reg_src = reg_is_k ? (size_t)kvh * p.page_size * kd + reg_c
                                    : (size_t)p.nkv * p.page_size * kd + (size_t)kvh * p.page_size * Dv + reg_c;
    auto load_tile = [&](int kbase, int buf) {
        __nv_bfloat16* Ks = Ks0 + buf * DAM_KEYS * QS;
        __nv_bfloat16* Vs = Vs0 + buf * DAM_KEYS * VS;
        const int nk = min(DAM_KEYS, hi - kbase + 1);
        if (regular) {
            // a thread keeps its 16-byte column of the key (or value) row and walks the keys: nothing but the page
            // lookup is worked out per copy
            __nv_bfloat16* dst = (reg_is_k ? Ks : Vs) + reg_dst;
            for (int key = reg_key0; key < nk; key += reg_step) {
                const int j = kbase + key, blk = j >> ps_shift;
                const int page = blk < p.max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= p.num_pages) { bad = true; continue; }
                cp_async16(dst + key * reg_stride, p.pool + (size_t)page * page_elems + reg_src + (size_t)(j & (p.page_size - 1)) * reg_row);
            }
            cp_async_commit();
            return;
        }
        const int perk = vec ? kd / 8 : kd, perv = vec ? Dv / 8 : Dv;
        for (int e = tid; e < nk * (perk + perv); e += 128) {
            const int key = e / (perk + perv), u = e - key * (perk + perv);
            const int j = kbase + key, blk = j / p.page_size;
            const int page = blk < p.max_blocks ? bt[blk] : -1;
            if (page < 0 || page >= p.num_pages) { bad = true; continue; }
            const __nv_bfloat16* pk = p.pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * kd;
            const __nv_bfloat16* pv = p.pool + (size_t)page * page_elems + (size_t)p.nkv * p.page_size * kd +
                                      ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * Dv;
            if (vec) {
                if (u < perk) {
                    const int c = u * 8, m = c / D, d = c - m * D;
                    cp_async16(Ks + key * QS + m * DP + d, pk + c);
                } else {
                    cp_async16(Vs + key * VS + (u - perk) * 8, pv + (u - perk) * 8);
                }
            } else if (u < perk) {
                const int m = u / D, d = u - m * D;
                Ks[key * QS + m * DP + d] = pk[u];
            } else {
                Vs[key * VS + (u - perk)] = pv[u - perk];
            }
        }
        cp_async_commit();
    };
    load_tile(lo, 0);
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += DAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * DAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * DAM_KEYS * VS;
        if (kbase + DAM_KEYS <= hi) {
            load_tile(kbase + DAM_KEYS, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = kbase + 16 * warp;                  // this warp's sixteen keys
        if (k0 <= hi)
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float S[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) S[i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DP / 16; ++ks) {
                uint32_t a[4];
                const __nv_bfloat16* qa = Qs + g * QS + m * DP + ks * 16 + 2 * t;
                a[0] = *reinterpret_cast<const uint32_t*>(qa);
                a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS);
                a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + 8);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const __nv_bfloat16* kb = Ks + (16 * warp + nt * 8 + g) * QS + m * DP + ks * 16 + 2 * t;
                    mma_bf16(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1, key = k0 + nt * 8 + 2 * t + (j & 1);
                    float sc;
                    if (p.cap > 0.0f) sc = fmaf(cap2, __fdividef(1.0f, exp2f(S[nt][j] * cap_in) + 1.0f), p.cap);
                    else sc = S[nt][j] * p.scale;
                    sc = (row_on[h] && key <= hi) ? sc : -INFINITY;
                    S[nt][j] = sc;
                    tmax[h] = fmaxf(tmax[h], sc);
                }
            float corr[2], mneg[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float mnew = fmaxf(mx[m][h], tmax[h]);
                corr[h] = mnew == -INFINITY ? 1.0f : exp2f((mx[m][h] - mnew) * LOG2E);
                mx[m][h] = mnew;
                mneg[h] = mnew == -INFINITY ? 0.0f : -mnew * LOG2E;
            }
            float tsum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float pr = exp2f(fmaf(S[nt][j], LOG2E, mneg[j >> 1]));
                    S[nt][j] = pr;
                    tsum[j >> 1] += pr;
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 1);
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 2);
                sm[m][h] = sm[m][h] * corr[h] + tsum[h];
            }
            uint32_t a[4];
            a[0] = pack_bf16(S[0][0], S[0][1]);
            a[1] = pack_bf16(S[0][2], S[0][3]);
            a[2] = pack_bf16(S[1][0], S[1][1]);
            a[3] = pack_bf16(S[1][2], S[1][3]);
#pragma unroll
            for (int nv = 0; nv < DVP / 8; ++nv) {
                O[m][nv][0] *= corr[0]; O[m][nv][1] *= corr[0];
                O[m][nv][2] *= corr[1]; O[m][nv][3] *= corr[1];
                uint32_t b0, b1;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (16 * warp + (lane & 15)) * VS + nv * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_bf16(O[m][nv], a, b0, b1);
            }
        }
        __syncthreads();
    }
    if (bad && lane == 0) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);
    // ---- the four warps' results into warp 0, in warp order (the stages are free: every copy has landed)
    float* sh = reinterpret_cast<float*>(dam_smem) + (size_t)tid * PER;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float* dst = sh + m * (DVP / 8 * 4 + 4);
        dst[0] = mx[m][0]; dst[1] = mx[m][1]; dst[2] = sm[m][0]; dst[3] = sm[m][1];
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[4 + i * 4 + j] = O[m][i][j];
    }
    __syncthreads();
    if (warp != 0) return;
    float inv[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float wgt[4][2], mstar[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = reinterpret_cast<float*>(dam_smem) + (size_t)(w * 32 + lane) * PER + m * (DVP / 8 * 4 + 4);
            mstar[0] = fmaxf(mstar[0], src[0]); mstar[1] = fmaxf(mstar[1], src[1]);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = reinterpret_cast<float*>(dam_smem) + (size_t)(w * 32 + lane) * PER + m * (DVP / 8 * 4 + 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                wgt[w][h] = src[h] == -INFINITY ? 0.0f : exp2f((src[h] - mstar[h]) * LOG2E);
                l[h] += src[2 + h] * wgt[w][h];
            }
        }
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float acc = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w)
                    acc = fmaf((reinterpret_cast<float*>(dam_smem) + (size_t)(w * 32 + lane) * PER + m * (DVP / 8 * 4 + 4))[4 + i * 4 + j],
                               wgt[w][j >> 1], acc);
                O[m][i][j] = acc;
            }
        inv[m][0] = l[0] > 0.0f ? 1.0f / l[0] : 0.0f;
        inv[m][1] = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    }
    float ss[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int h = j >> 1;
            const float o = O[0][i][j] * inv[0][h] - p.lambda * (O[1][i][j] * inv[1][h]);
            O[0][i][j] = o;
            ss[h] = fmaf(o, o, ss[h]);
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
        ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
        if (!row_on[h]) continue;
        const float nrm = p.out_scale / sqrtf(ss[h] / (float)Dv + p.eps);
        __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + (size_t)(kvh * G + g + 8 * h) * Dv;
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i) {
            const int c = i * 8 + 2 * t;
            if (c < Dv) dst[c] = __float2bfloat16_rn(O[0][i][2 * h] * nrm);
            if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[0][i][2 * h + 1] * nrm);
        }
    }
}

template <int DP, int DVP>
static int dag_launch(const DamParams& p, cudaStream_t stream) {
    const size_t tiles = (size_t)((16 + 2 * DAM_KEYS) * (2 * DP + DAM_PAD) + 2 * DAM_KEYS * (DVP + DAM_PAD)) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)128 * (2 * (DVP / 8 * 4 + 4) + 1) * sizeof(float);
    const size_t smem = tiles > merge ? tiles : merge;
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(diff_attention_group_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(diff_attention_group_kernel<DP, DVP>, dim3(p.nkv, p.num_reqs), dim3(128), smem, stream, p);
    return airun_launch_status();
}

template <int DP, int DVP>
static int dam_launch(const DamParams& p, int max_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(3 * DAM_ROWS * (2 * DP + DAM_PAD) + 2 * DAM_KEYS * (DVP + DAM_PAD)) * sizeof(__nv_bfloat16);
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(diff_attention_mma_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (max_tiles > 65535) return AIRUN_ERR_ARG;
    airun_launch(diff_attention_mma_kernel<DP, DVP>, dim3(p.nh, max_tiles), dim3(128), smem, stream, p);
    return airun_launch_status();
}

// max_tiles: an upper bound of the number of 64-token tiles of the batch, e.g. ceil(T / 64) + requests.
AIRUN_EXPORT int airun_diff_attention_mma(const void* q, void* out, long long out_stride, const void* pool,
                                          const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                          const int32_t* context_lens, int num_reqs, int max_tiles, int num_pages,
                                          int page_size, int nh, int nkv, int D, int Dv, float scale, float cap, int chunk,
                                          int window, float lambda, float eps, float out_scale, int skip_single, int* err,
                                          cudaStream_t stream) {
    if (num_reqs < 0 || max_tiles < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 128 || Dv <= 0 || Dv > 128 ||
        page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || chunk < 0 || window < 0 || !err || nh > 65535 ||
        out_stride < (long long)nh * Dv || !cu_tokens || !context_lens)
        return AIRUN_ERR_ARG;
    if (num_reqs == 0 || max_tiles == 0) return AIRUN_OK;
    DamParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.pool = (const __nv_bfloat16*)pool; p.block_table = block_table; p.max_blocks = max_blocks;
    p.cu_tokens = cu_tokens; p.context_lens = context_lens; p.num_reqs = num_reqs; p.num_pages = num_pages;
    p.page_size = page_size; p.nh = nh; p.nkv = nkv; p.D = D; p.Dv = Dv; p.scale = scale; p.cap = cap;
    p.lambda = lambda; p.eps = eps; p.out_scale = out_scale; p.chunk = chunk; p.window = window; p.skip_single = skip_single; p.err = err;
    const int dp = D <= 32 ? 32 : D <= 64 ? 64 : 128, dvp = Dv <= 32 ? 32 : Dv <= 64 ? 64 : 128;
#define DAM_CASE(A, B) if (dp == A && dvp == B) return dam_launch<A, B>(p, max_tiles, stream)
    DAM_CASE(32, 32); DAM_CASE(32, 64); DAM_CASE(32, 128);
    DAM_CASE(64, 32); DAM_CASE(64, 64); DAM_CASE(64, 128);
    DAM_CASE(128, 32); DAM_CASE(128, 64); DAM_CASE(128, 128);
#undef DAM_CASE
    return AIRUN_ERR_UNSUPPORTED;
}

// The single tokens of the batch on the tensor cores (groups of up to 16 query heads a KV head, D and Dv up to 128).
AIRUN_EXPORT int airun_diff_attention_group(const void* q, void* out, long long out_stride, const void* pool,
                                            const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                            const int32_t* context_lens, int num_reqs, int num_pages, int page_size,
                                            int nh, int nkv, int D, int Dv, float scale, float cap, int chunk, int window,
                                            float lambda, float eps, float out_scale, int* err, cudaStream_t stream) {
    if (num_reqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || D <= 0 || D > 128 || Dv <= 0 || Dv > 128 ||
        page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || chunk < 0 || window < 0 || !err || num_reqs > 65535 ||
        out_stride < (long long)nh * Dv || !cu_tokens || !context_lens)
        return AIRUN_ERR_ARG;
    if (num_reqs == 0) return AIRUN_OK;
    DamParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.pool = (const __nv_bfloat16*)pool; p.block_table = block_table; p.max_blocks = max_blocks;
    p.cu_tokens = cu_tokens; p.context_lens = context_lens; p.num_reqs = num_reqs; p.num_pages = num_pages;
    p.page_size = page_size; p.nh = nh; p.nkv = nkv; p.D = D; p.Dv = Dv; p.scale = scale; p.cap = cap;
    p.lambda = lambda; p.eps = eps; p.out_scale = out_scale; p.chunk = chunk; p.window = window; p.skip_single = 0;
    p.err = err;
    const int dp = D <= 32 ? 32 : D <= 64 ? 64 : 128, dvp = Dv <= 32 ? 32 : Dv <= 64 ? 64 : 128;
#define DAG_CASE(A, B) if (dp == A && dvp == B) return dag_launch<A, B>(p, stream)
    DAG_CASE(32, 32); DAG_CASE(32, 64); DAG_CASE(32, 128);
    DAG_CASE(64, 32); DAG_CASE(64, 64); DAG_CASE(64, 128);
    DAG_CASE(128, 32); DAG_CASE(128, 64); DAG_CASE(128, 128);
#undef DAG_CASE
    return AIRUN_ERR_UNSUPPORTED;
}
