// Attention over a cached latent: every token caches ONE row [c (R values) | kr (rd values)] that all heads share,
// c being the normed down-projection of the layer's input and kr a rotated key part.  Head h's key for a cached
// token is (Wuk_h c, kr) and its value Wuv_h c, so with the query's unrotated part carried into the latent space,
//     qa_h = Wuk_h^T qn_h            (R values),
// the score is  s = scale * (qa_h . c + qr_h . kr),  the weighted sum of values is Wuv_h (sum_j p_j c_j), and the
// cache is read as it is: the up-projections are applied to the query and to the result, never to the cache.
// A query at position i sees keys j with 0 <= i - j < window (window 0: all j <= i).  The softmax denominator holds one
// more term exp(sink_h), a learnt number per head with no key and no value.  Scores, weights, norms, positions and
// angles are float32; queries, cached rows and results are stored in the compute type.
//
// Rotation: pair (2i, 2i + 1) of the rotated part turns by pos * inv_freq[i]; cos and sin are both multiplied by
// `rot_mult` (a stretched rotation that goes with scaled frequencies).  inv_freq comes from the host.
#include "common.cuh"

// One block per token.  proj [T][stride] float32 holds [dq (q_rank) | dkv (R) | kr (rd)]; the last two only when
// `store`.  cq = dq / rms(dq) * wq in the compute type; the cache row = [dkv / rms(dkv) * wkv | rotate(kr)].
template <typename TC>
__global__ __launch_bounds__(256) void latent_prepare_kernel(
    const float* __restrict__ proj, long long stride, const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
    TC* __restrict__ cq, int q_rank, int R, int rd, int rot_dims, const float* __restrict__ inv_freq, float rot_mult,
    TC* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int store, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int req = req_of_token[t], pos = positions[t];
    if (req < 0 || pos < 0) return;
    if (req >= num_reqs) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ); return; }
    const float* row = proj + (size_t)t * stride;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, red);
    const float inv_q = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f32<TC>(row[i] * inv_q * wq[i]);
    if (!store) return;
    const int blk = pos / page_size;
    const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) { if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE); return; }
    TC* dst = pool + ((size_t)page * page_size + (pos % page_size)) * (R + rd);
    const float* c = row + q_rank;
    ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
    ss = block_sum(ss, red);
    const float inv_c = 1.0f / sqrtf(ss / (float)R + eps);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<TC>(c[i] * inv_c * wkv[i]);
    const float* kr = c + R;
    for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) {
        const float a = kr[2 * i], b = kr[2 * i + 1];
        if (2 * i + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= rot_mult; cs *= rot_mult;
            dst[R + 2 * i] = from_f32<TC>(a * cs - b * sn);
            dst[R + 2 * i + 1] = from_f32<TC>(b * cs + a * sn);
        } else {
            dst[R + 2 * i] = from_f32<TC>(a);
            dst[R + 2 * i + 1] = from_f32<TC>(b);
        }
    }
    if ((rd & 1) && threadIdx.x == 0) dst[R + rd - 1] = from_f32<TC>(kr[rd - 1]);
}

AIRUN_EXPORT int airun_latent_prepare(const float* proj, long long stride, const float* wq, const float* wkv, float eps, void* cq,
                                      int dtype, int q_rank, int R, int rd, int rot_dims, const float* inv_freq, float rot_mult,
                                      void* pool, const int32_t* block_table, int max_blocks, const int32_t* positions,
                                      const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size, int store,
                                      int* err, cudaStream_t stream) {
    if (T < 0 || q_rank <= 0 || R <= 0 || rd < 0 || rot_dims < 0 || rot_dims > rd || (rot_dims & 1) || !wq || !err ||
        (store && (!pool || !block_table || !wkv || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)) || (rot_dims > 0 && !inv_freq))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
#define LAUNCH(TC) airun_launch(latent_prepare_kernel<TC>, dim3(T), dim3(256), 0, stream, proj, stride, wq, wkv, eps, (TC*)cq, q_rank, R, rd, \
        rot_dims, inv_freq, rot_mult, (TC*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, store, err)
    if (dtype == AIRUN_DT_F32) LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}

// q [T][H][D + rd] float32 (the up-projected query, head by head [unrotated | rotated part]) ->
// qn [T][H][D] in the compute type, and the rotated part, turned by the token's position, into
// qlat[t][h][R .. R + rd) (qlat rows are [H][R + rd]; the first R of each head are filled by the product with Wuk^T).
template <typename TC>
__global__ __launch_bounds__(256) void latent_query_kernel(
    const float* __restrict__ q, TC* __restrict__ qn, TC* __restrict__ qlat, int H, int D, int R, int rd, int rot_dims,
    const float* __restrict__ inv_freq, float rot_mult, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (req_of_token[t] < 0 || pos < 0) return;
    const float* row = q + (size_t)t * H * (D + rd);
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
        const int h = e / D, d = e - h * D;
        qn[(size_t)t * H * D + e] = from_f32<TC>(row[(size_t)h * (D + rd) + d]);
    }
    const int half = (rd + 1) / 2;
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float* src = row + (size_t)h * (D + rd) + D;
        TC* dst = qlat + ((size_t)t * H + h) * (R + rd) + R;
        if (2 * i + 1 >= rd) { dst[2 * i] = from_f32<TC>(src[2 * i]); continue; }
        const float a = src[2 * i], b = src[2 * i + 1];
        if (2 * i + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= rot_mult; cs *= rot_mult;
            dst[2 * i] = from_f32<TC>(a * cs - b * sn);
            dst[2 * i + 1] = from_f32<TC>(b * cs + a * sn);
        } else {
            dst[2 * i] = from_f32<TC>(a);
            dst[2 * i + 1] = from_f32<TC>(b);
        }
    }
}

AIRUN_EXPORT int airun_latent_query(const float* q, void* qn, void* qlat, int dtype, int T, int H, int D, int R, int rd, int rot_dims,
                                    const float* inv_freq, float rot_mult, const int32_t* positions, const int32_t* req_of_token,
                                    cudaStream_t stream) {
    if (T < 0 || H <= 0 || D <= 0 || R <= 0 || rd < 0 || rot_dims < 0 || rot_dims > rd || (rot_dims & 1) || (rot_dims > 0 && !inv_freq))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
#define LAUNCH(TC) airun_launch(latent_query_kernel<TC>, dim3(T), dim3(256), 0, stream, q, (TC*)qn, (TC*)qlat, H, D, R, rd, rot_dims, inv_freq, \
        rot_mult, positions, req_of_token)
    if (dtype == AIRUN_DT_F32) LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}

// The plain attention: one block per (token, head), float32 arithmetic.  Each warp walks every LAT_WARPS-th visible
// cached row with a running maximum and sum, lanes hold the row's elements; the warps' results are merged at the
// end together with the sink's term.  out[t][h] = sum_j p_j c_j (R values) in the compute type.
#define LAT_WARPS 4
#define LAT_PER_LANE 20      // R + rd <= 640
template <typename TC>
__global__ __launch_bounds__(32 * LAT_WARPS) void latent_attention_kernel(
    const TC* __restrict__ qlat, TC* __restrict__ out, const TC* __restrict__ pool, const int32_t* __restrict__ block_table,
    int max_blocks, const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages,
    int page_size, int H, int R, int rd, float scale, int window, const float* __restrict__ sink, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* s_max = smem;
    float* s_sum = smem + LAT_WARPS;
    float* s_acc = smem + 2 * LAT_WARPS;
    const int t = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t], req = req_of_token[t];
    const int KD = R + rd;
    TC* dst = out + ((size_t)t * H + head) * R;
    if (req < 0 || pos < 0 || req >= num_reqs) {
        if (req >= num_reqs && threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = from_f32<TC>(0.0f);
        return;
    }
    const TC* qv = qlat + ((size_t)t * H + head) * KD;
    float qreg[LAT_PER_LANE], acc[LAT_PER_LANE];
#pragma unroll
    for (int i = 0; i < LAT_PER_LANE; ++i) {
        const int d = lane + i * 32;
        qreg[i] = d < KD ? to_f32<TC>(qv[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float run_max = -INFINITY, run_sum = 0.0f;
    const int32_t* bt = block_table + (size_t)req * max_blocks;
    const int begin = window > 0 ? max(0, pos - window + 1) : 0;
    bool bad = false;
    for (int j = begin + warp; j <= pos; j += LAT_WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const TC* kj = pool + ((size_t)page * page_size + (j % page_size)) * KD;
        float kreg[LAT_PER_LANE];
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < LAT_PER_LANE; ++i) {
            const int d = lane + i * 32;
            kreg[i] = d < KD ? to_f32<TC>(kj[d]) : 0.0f;
            dot = fmaf(qreg[i], kreg[i], dot);
        }
        dot = warp_sum(dot) * scale;
        const float new_max = fmaxf(run_max, dot);
        const float corr = expf(run_max - new_max);
        const float p = expf(dot - new_max);
        run_sum = run_sum * corr + p;
#pragma unroll
        for (int i = 0; i < LAT_PER_LANE; ++i) acc[i] = fmaf(p, kreg[i], acc[i] * corr);
        run_max = new_max;
    }
    if (bad && lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
    if (lane == 0) { s_max[warp] = run_max; s_sum[warp] = run_sum; }
#pragma unroll
    for (int i = 0; i < LAT_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < R) s_acc[(size_t)warp * R + d] = acc[i];
    }
    __syncthreads();
    if (warp != 0) return;
    const float sk = sink ? sink[head] : -INFINITY;
    float gmax = sk;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) gmax = fmaxf(gmax, s_max[w]);
    float weight[LAT_WARPS], gsum = sink ? expf(sk - gmax) : 0.0f;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) {
        weight[w] = s_sum[w] > 0.0f ? expf(s_max[w] - gmax) : 0.0f;
        gsum += s_sum[w] * weight[w];
    }
    const float inv = gsum > 0.0f ? 1.0f / gsum : 0.0f;
    for (int d = lane; d < R; d += 32) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < LAT_WARPS; ++w) v = fmaf(s_acc[(size_t)w * R + d], weight[w], v);
        dst[d] = from_f32<TC>(v * inv);
    }
}

AIRUN_EXPORT int airun_latent_attention(const void* qlat, void* out, int dtype, const void* pool, const int32_t* block_table,
                                        int max_blocks, const int32_t* positions, const int32_t* req_of_token, int T, int num_reqs,
                                        int num_pages, int page_size, int H, int R, int rd, float scale, int window,
                                        const float* sink, int* err, cudaStream_t stream) {
    if (T < 0 || H <= 0 || H > 65535 || R <= 0 || rd < 0 || R + rd > 32 * LAT_PER_LANE || page_size <= 0 || num_pages <= 0 ||
        max_blocks <= 0 || window < 0 || !err)
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const size_t smem = (size_t)LAT_WARPS * (2 + R) * sizeof(float);
#define LAUNCH(TC) airun_launch(latent_attention_kernel<TC>, dim3(T, H), dim3(32 * LAT_WARPS), smem, stream, (const TC*)qlat, (TC*)out, \
        (const TC*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, H, R, rd, scale, window, sink, err)
    if (dtype == AIRUN_DT_F32) LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}
