// Attention over a cached latent on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums).
//
// The formulas are those of latent_attention.cu: every cached row [c (R) | kr (rd)] is key AND value for all heads,
// s = scale * q_lat . row, a sliding window, a sink in the softmax's denominator, out = sum_j p_j c_j.  Because all
// heads share the rows, the rows of a product tile are (token, head) pairs: a CTA takes TOK consecutive tokens of
// one request times up to 16 * RW heads (RW row tiles of 16), reads every cached row the tokens see ONCE for all of
// them, and keeps 256 of the R output columns in registers (blockIdx.z picks the columns; the scores are computed
// again for every 256 columns, which is cheaper than a second trip of the probabilities through shared memory).
//
//   prompt portions: 8 (or 4) warps = as many row tiles, key tiles of 32 rows, every warp takes all keys of a tile,
//                    tiles arrive by cp.async in two stages (the next one is on its way while this one is used);
//   single tokens:   one row tile, key tiles of 128 rows of which each of the 8 warps takes 16, one stage; the warps'
//                    (maximum, sum, output) are merged through shared memory at the end, in warp order.
// A cached row is found through the request's block table.  A group of TOK batch rows that straddles two requests is handled
// request by request.  Every row keeps its own maximum and sum, so a token's result does not depend on the batch.
#include "common.cuh"

#define LM_CW 256                 // output columns of a CTA
#define LM_NT (LM_CW / 8)

__device__ __forceinline__ void lm_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
// ldmatrix on shared-memory addresses that are worked out once a tile and stepped by plain adds
__device__ __forceinline__ uint32_t lm_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldsm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

struct LatentMmaArgs {
    const __nv_bfloat16* qlat; __nv_bfloat16* out; const __nv_bfloat16* pool;
    const int32_t* block_table; int max_blocks;
    const int32_t* positions; const int32_t* req_of_token;
    int T, num_reqs, num_pages, page_size, H, R, rd, window;
    float scale_log2;             // scale * log2(e)
    const float* sink;
    int hg, tok;                  // heads of a CTA, tokens of a CTA
    int kd16, kdp;                // the row padded to k-steps of 16; the shared-memory row stride in elements
    int* err;
};

template <int RW, int KW, int STAGES>
__global__ __launch_bounds__(32 * RW * KW, 1) void latent_attention_mma_kernel(LatentMmaArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int NWARP = RW * KW, NTHREAD = 32 * NWARP;
    constexpr int BN = KW == 1 ? 32 : 16 * KW;   // cached rows of a tile
    constexpr int WK = BN / KW;                  // cached rows of a tile one warp takes
    constexpr int ROWS = 16 * RW;
    extern __shared__ __align__(16) uint8_t lm_smem[];
    __nv_bfloat16* s_q = reinterpret_cast<__nv_bfloat16*>(lm_smem);                  // [ROWS][kdp]
    __nv_bfloat16* s_k = s_q + (size_t)ROWS * a.kdp;                                 // [2][BN][kdp]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rw = KW == 1 ? warp : 0, kw = KW == 1 ? 0 : warp;
    const int KD = a.R + a.rd, kdp = a.kdp;
    const int t0 = blockIdx.x * a.tok, t1 = min(t0 + a.tok, a.T);
    const int h0 = blockIdx.y * a.hg, c0 = blockIdx.z * LM_CW;
    const int g = lane >> 2, qd = lane & 3;
    const int chunks = KD / 8;                  // 16-byte pieces of a cached row

    for (int tb = t0; tb < t1;) {
        const int req = a.req_of_token[tb];
        int te = tb + 1;
        if (req < 0 || req >= a.num_reqs) {
            if (req >= a.num_reqs && threadIdx.x == 0) atomicOr(a.err, AIRUN_DEV_BAD_REQ);
            tb = te;
            continue;
        }
        while (te < t1 && a.req_of_token[te] == req) ++te;
        const int p_first = a.positions[tb], n_tok = te - tb;
        const int p_last = p_first + n_tok - 1;
        const int j_lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
        const int tile0 = j_lo / BN, tile_end = p_last / BN + 1;
        const int32_t* bt = a.block_table + (size_t)req * a.max_blocks;
        __syncthreads();                         // the pass before is done with the shared memory
        // the padding behind a cached row's last element is zero in every stage; the tile loads never copy into it
        for (int e = threadIdx.x; e < STAGES * BN * (kdp / 8 - chunks); e += NTHREAD) {
            const int row = e / (kdp / 8 - chunks), ch = chunks + e - row * (kdp / 8 - chunks);
            *reinterpret_cast<uint4*>(s_k + (size_t)row * kdp + ch * 8) = make_uint4(0, 0, 0, 0);
        }
        // the queries: row r = (token r / hg, head h0 + r % hg); rows beyond the group and the padding are zero
        for (int r = warp; r < ROWS; r += NWARP) {            // a warp a row: what the row needs is worked out once
            const int tl = r / a.hg, h = h0 + r - tl * a.hg;
            const bool on = tl < n_tok && h < a.H;
            const __nv_bfloat16* src = a.qlat + ((size_t)(tb + (on ? tl : 0)) * a.H + (on ? h : 0)) * KD;
            for (int ch = lane; ch < kdp / 8; ch += 32) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (on && ch < chunks) v = *reinterpret_cast<const uint4*>(src + ch * 8);
                *reinterpret_cast<uint4*>(s_q + (size_t)r * kdp + ch * 8) = v;
            }
        }
        bool bad = false;
        auto load_tile = [&](int tile, int buf) {
            __nv_bfloat16* dst = s_k + (size_t)buf * BN * kdp;
            for (int kr = warp; kr < BN; kr += NWARP) {        // a warp a cached row: one page lookup for the whole row
                const int j = tile * BN + kr;
                const int blk = j / a.page_size;
                int page = -1;
                if (j <= p_last && j >= j_lo && blk < a.max_blocks) {
                    page = bt[blk];
                    if (page >= a.num_pages) { bad = true; page = -1; }
                }
                __nv_bfloat16* d = dst + (size_t)kr * kdp;
                if (page >= 0) {
                    const __nv_bfloat16* src = a.pool + ((size_t)page * a.page_size + (j - blk * a.page_size)) * KD;
                    for (int ch = lane; ch < chunks; ch += 32) lm_cp16(d + ch * 8, src + ch * 8);
                } else {
                    for (int ch = lane; ch < chunks; ch += 32) *reinterpret_cast<uint4*>(d + ch * 8) = make_uint4(0, 0, 0, 0);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (STAGES == 2) load_tile(tile0, 0);

        float o[LM_NT][4];
#pragma unroll
        for (int i = 0; i < LM_NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
        // the two rows of this thread: rw * 16 + g and + 8; their positions
        int pos_r[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = rw * 16 + g + 8 * i, tl = r / a.hg;
            pos_r[i] = (tl < n_tok && h0 + r - tl * a.hg < a.H) ? p_first + tl : -1;       // -1: the row sees nothing
        }
        const int n_pairs = min(LM_NT / 2, (a.R - c0 + 15) / 16);      // pairs of 8 output columns this CTA has

        for (int tile = tile0, it = 0; tile < tile_end; ++tile, ++it) {
            const int buf = STAGES == 2 ? (it & 1) : 0;
            if (STAGES == 2 && tile + 1 < tile_end) {
                load_tile(tile + 1, buf ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                if (STAGES == 1) load_tile(tile, 0);       // one stage: the warps of a tile wait for it together
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            const __nv_bfloat16* kt = s_k + (size_t)buf * BN * kdp + (size_t)kw * WK * kdp;
            // S = Q K^T for this warp's 16 rows and WK cached rows
            float s[WK / 8][4];
#pragma unroll
            for (int i = 0; i < WK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
            uint32_t qaddr = lm_saddr(s_q + (size_t)(rw * 16 + (lane & 15)) * kdp + (lane >> 4) * 8);
            uint32_t kaddr = lm_saddr(kt + (size_t)((lane & 7) + ((lane >> 4) << 3)) * kdp + ((lane >> 3) & 1) * 8);
            const uint32_t kstep = (uint32_t)(16 * kdp * 2);
#pragma unroll 4
            for (int k0 = 0; k0 < a.kd16; k0 += 16, qaddr += 32, kaddr += 32) {
                uint32_t af[4];
                lm_ldsm4(af, qaddr);
#pragma unroll
                for (int np = 0; np < WK / 16; ++np) {
                    uint32_t bf[4];
                    lm_ldsm4(bf, kaddr + np * kstep);
                    lm_mma(s[2 * np], af, bf[0], bf[1]);
                    lm_mma(s[2 * np + 1], af, bf[2], bf[3]);
                }
            }
            // scale, mask, online softmax (base 2)
            const int jbase = tile * BN + kw * WK + qd * 2;
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < WK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1, j = jbase + nt * 8 + (e & 1);
                    const bool vis = j <= pos_r[i] && j >= j_lo && (a.window == 0 || pos_r[i] - j < a.window);
                    const float v = vis ? s[nt][e] * a.scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    tmax[i] = fmaxf(tmax[i], v);
                }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
                tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
                const float m_new = fmaxf(m_run[i], tmax[i]);
                corr[i] = m_new == -INFINITY ? 1.0f : exp2f(m_run[i] - m_new);
                m_run[i] = m_new;
            }
            float psum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int nt = 0; nt < WK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const float p = m_run[i] == -INFINITY ? 0.0f : exp2f(s[nt][e] - m_run[i]);
                    s[nt][e] = p;
                    psum[i] += p;
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 1);
                psum[i] += __shfl_xor_sync(0xffffffffu, psum[i], 2);
                l_run[i] = l_run[i] * corr[i] + psum[i];
            }
            if (corr[0] != 1.0f || corr[1] != 1.0f) {       // once the maxima have settled nothing is rescaled
#pragma unroll
                for (int i = 0; i < LM_NT; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
            }
            // O += P V, V = the first R elements of the same cached rows
            const uint32_t vaddr = lm_saddr(kt + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * kdp + c0 + (lane >> 4) * 8);
#pragma unroll
            for (int ks = 0; ks < WK / 16; ++ks) {
                uint32_t pf[4] = {lm_pack(s[2 * ks][0], s[2 * ks][1]), lm_pack(s[2 * ks][2], s[2 * ks][3]),
                                  lm_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]), lm_pack(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
                for (int np = 0; np < LM_NT / 2; ++np) {
                    if (np < n_pairs) {
                        uint32_t vf[4];
                        lm_ldsm4t(vf, vaddr + ks * kstep + np * 32);
                        lm_mma(o[2 * np], pf, vf[0], vf[1]);
                        lm_mma(o[2 * np + 1], pf, vf[2], vf[3]);
                    }
                }
            }
            __syncthreads();                     // everybody is done with this stage before it is loaded again
        }
        if (bad && lane == 0) atomicOr(a.err, AIRUN_DEV_BAD_PAGE);

        if (KW > 1) {
            // merge the warps' partial results of the same 16 rows, in warp order, through shared memory
            float* s_m = reinterpret_cast<float*>(s_k);                 // [KW][16] maxima, [KW][16] sums, then [KW][16][LM_CW]
            float* s_l = s_m + KW * 16;
            float* s_o = s_l + KW * 16;
            if (qd == 0) {
                s_m[warp * 16 + g] = m_run[0]; s_m[warp * 16 + g + 8] = m_run[1];
                s_l[warp * 16 + g] = l_run[0]; s_l[warp * 16 + g + 8] = l_run[1];
            }
#pragma unroll
            for (int nt = 0; nt < LM_NT; ++nt) {
                float* d = s_o + ((size_t)warp * 16 + g) * LM_CW + nt * 8 + qd * 2;
                d[0] = o[nt][0]; d[1] = o[nt][1];
                d[8 * LM_CW] = o[nt][2]; d[8 * LM_CW + 1] = o[nt][3];
            }
            __syncthreads();
            // thread t handles row t / 8 and every 8th column from t % 8
            const int r = threadIdx.x >> 3, cs = threadIdx.x & 7;
            const int tl = r / a.hg, h = h0 + r - tl * a.hg;
            if (r < 16 && tl < n_tok && h < a.H) {
                float gm = a.sink ? a.sink[h] * 1.4426950408889634f : -INFINITY;
                const float sk = gm;
#pragma unroll
                for (int w = 0; w < KW; ++w) gm = fmaxf(gm, s_m[w * 16 + r]);
                float wgt[KW], gl = a.sink ? exp2f(sk - gm) : 0.0f;
#pragma unroll
                for (int w = 0; w < KW; ++w) {
                    wgt[w] = s_m[w * 16 + r] == -INFINITY ? 0.0f : exp2f(s_m[w * 16 + r] - gm);
                    gl += s_l[w * 16 + r] * wgt[w];
                }
                const float inv = gl > 0.0f ? 1.0f / gl : 0.0f;
                __nv_bfloat16* dst = a.out + ((size_t)(tb + tl) * a.H + h) * a.R;
                for (int c = cs; c < LM_CW && c0 + c < a.R; c += 8) {
                    float v = 0.0f;
#pragma unroll
                    for (int w = 0; w < KW; ++w) v = fmaf(s_o[((size_t)w * 16 + r) * LM_CW + c], wgt[w], v);
                    dst[c0 + c] = __float2bfloat16_rn(v * inv);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = rw * 16 + g + 8 * i, tl = r / a.hg, h = h0 + r - tl * a.hg;
                if (tl >= n_tok || h >= a.H) continue;
                float m = m_run[i], l = l_run[i], scale_o = 1.0f;
                if (a.sink) {
                    const float sk = a.sink[h] * 1.4426950408889634f;
                    const float mf = fmaxf(m, sk);
                    scale_o = m == -INFINITY ? 0.0f : exp2f(m - mf);
                    l = l * scale_o + exp2f(sk - mf);
                }
                const float inv = l > 0.0f ? scale_o / l : 0.0f;
                __nv_bfloat16* dst = a.out + ((size_t)(tb + tl) * a.H + h) * a.R + c0;
#pragma unroll
                for (int nt = 0; nt < LM_NT; ++nt) {
                    const int c = nt * 8 + qd * 2;
                    if (c0 + c < a.R) dst[c] = __float2bfloat16_rn(o[nt][2 * i] * inv);
                    if (c0 + c + 1 < a.R) dst[c + 1] = __float2bfloat16_rn(o[nt][2 * i + 1] * inv);
                }
            }
        }
        tb = te;
    }
}

// qlat [T][H][R + rd], out [T][H][R], pool pages of [page_size][R + rd], all bfloat16.  ``single``: the step's rows
// are mostly single tokens of different requests (one token a CTA, the warps share the keys); otherwise prompt
// portions (several tokens a CTA).  Needs (R + rd) % 8 == 0.
AIRUN_EXPORT int airun_latent_attention_mma(const void* qlat, void* out, const void* pool, const int32_t* block_table,
                                            int max_blocks, const int32_t* positions, const int32_t* req_of_token, int T,
                                            int num_reqs, int num_pages, int page_size, int H, int R, int rd, float scale,
                                            int window, const float* sink, int single, int* err, cudaStream_t stream) {
    const int KD = R + rd;
    if (T < 0 || H <= 0 || R <= 0 || rd < 0 || KD % 8 != 0 || KD > 1024 || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
        window < 0 || !err || (((uintptr_t)qlat | (uintptr_t)pool) & 15))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    LatentMmaArgs a = {};
    a.qlat = (const __nv_bfloat16*)qlat; a.out = (__nv_bfloat16*)out; a.pool = (const __nv_bfloat16*)pool;
    a.block_table = block_table; a.max_blocks = max_blocks; a.positions = positions; a.req_of_token = req_of_token;
    a.T = T; a.num_reqs = num_reqs; a.num_pages = num_pages; a.page_size = page_size; a.H = H; a.R = R; a.rd = rd; a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.sink = sink; a.err = err;
    a.kd16 = (KD + 15) / 16 * 16;
    a.kdp = a.kd16 + 8;
    // prompt portions: 8 row tiles (128 rows) a CTA when its queries and two key tiles fit the shared memory, else 4;
    // single tokens: one row tile, 8 warps on the 128 cached rows of a tile, one stage
    const size_t limit = 227 * 1024;
    int rw = single ? 1 : 8;
    if (!single && ((size_t)128 + 2 * 32) * a.kdp * 2 > limit) rw = 4;
    const int rows = 16 * rw, bn = single ? 128 : 32, stages = single ? 1 : 2;
    a.hg = H < rows ? H : rows;
    a.tok = rows / a.hg;
    size_t kbytes = (size_t)stages * bn * a.kdp * 2;
    if (single) { const size_t merge = (2 * 8 * 16 + (size_t)8 * 16 * LM_CW) * 4; if (kbytes < merge) kbytes = merge; }
    const size_t smem = (size_t)rows * a.kdp * 2 + kbytes;
    if (smem > limit) return AIRUN_ERR_ARG;
    dim3 grid(ceil_div_i(T, a.tok), ceil_div_i(H, a.hg), ceil_div_i(R, LM_CW));
    if (grid.y > 65535 || grid.z > 65535) return AIRUN_ERR_ARG;
    static unsigned long long conf1 = 0, conf4 = 0, conf8 = 0;
#define LM_LAUNCH(RW_, KW_, ST_, CONF) do { \
        auto kern = latent_attention_mma_kernel<RW_, KW_, ST_>; \
        if (first_on_device(CONF)) { \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit); \
            if (e != cudaSuccess) return (int)e; \
        } \
        airun_launch(kern, grid, dim3(32 * RW_ * KW_), smem, stream, a); } while (0)
    if (single) LM_LAUNCH(1, 8, 1, conf1);
    else if (rw == 8) LM_LAUNCH(8, 1, 2, conf8);
    else LM_LAUNCH(4, 1, 2, conf4);
#undef LM_LAUNCH
    return airun_launch_status();
}
