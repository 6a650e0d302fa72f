// Differential attention over cache pages: two softmax attention maps per head over the same values,
// combined as a difference.
//
// Query head h carries two query vectors of size D (map 1 in its first D columns, map 2 in the next D)
// and reads KV head h / (heads / kv_heads), whose key row holds two key vectors laid out the same way
// and one value vector of size Dv.  For each map m:
//     s_m[j] = scale * (q_m . k_m[j]);  with a cap c > 0:  s_m[j] <- c * tanh(s_m[j] / c);
//     a_m = softmax over the visible keys j of s_m, applied to the values.
// Key j is visible to the query at position i iff j <= i, and, with chunk C > 0, j / C == i / C (chunks
// are counted from position 0 of the sequence), and, with window w > 0, i - j < w.  Then
//     o = a_1 - lambda * a_2;   o <- o / sqrt(mean(o^2) + eps) * out_scale        (per head, over Dv).
// lambda, eps and out_scale are numbers of the layer.  Scores, softmax, the difference and the norm
// are float32; q, keys and values are read in their storage type.
//
// A page of the cache holds, for `page_size` tokens, the keys of all KV heads ([kv_heads][page_size][2D])
// followed by the values ([kv_heads][page_size][Dv]).
#include "common.cuh"

#define DA_WARPS 4
#define DA_MAX_PER_LANE 8     // D <= 256 and Dv <= 256

// q_out = proj[:, :q_width] + q_bias in the storage type; keys and values (with their biases) into the
// token's page.  One block per token.
template <typename T>
__global__ void qkv_bias_store_kernel(const float* __restrict__ proj, long long proj_stride,
                                      const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                      const float* __restrict__ v_bias, T* __restrict__ q_out, T* __restrict__ pool,
                                      const int32_t* __restrict__ block_table, int max_blocks,
                                      const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token,
                                      int num_reqs, int num_pages, int page_size, int q_width, int nkv, int kd, int vd,
                                      int store, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int req = req_of_token[t], pos = positions[t];
    if (req < 0 || pos < 0) return;
    if (req >= num_reqs) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        return;
    }
    const float* row = proj + (size_t)t * proj_stride;
    for (int c = threadIdx.x; c < q_width; c += blockDim.x)
        q_out[(size_t)t * q_width + c] = from_f32<T>(row[c] + (q_bias ? q_bias[c] : 0.0f));
    if (!store) return;
    const int blk = pos / page_size, slot = pos - blk * page_size;
    const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
        return;
    }
    T* pk = pool + (size_t)page * nkv * page_size * (kd + vd);
    T* pv = pk + (size_t)nkv * page_size * kd;
    const float* krow = row + q_width;
    const float* vrow = krow + nkv * kd;
    for (int c = threadIdx.x; c < nkv * kd; c += blockDim.x) {
        const int g = c / kd, e = c - g * kd;
        pk[((size_t)g * page_size + slot) * kd + e] = from_f32<T>(krow[c] + (k_bias ? k_bias[c] : 0.0f));
    }
    for (int c = threadIdx.x; c < nkv * vd; c += blockDim.x) {
        const int g = c / vd, e = c - g * vd;
        pv[((size_t)g * page_size + slot) * vd + e] = from_f32<T>(vrow[c] + (v_bias ? v_bias[c] : 0.0f));
    }
}

AIRUN_EXPORT int airun_qkv_bias_store(const float* proj, long long proj_stride, const float* q_bias, const float* k_bias,
                                      const float* v_bias, void* q_out, void* pool, int dtype,
                                      const int32_t* block_table, int max_blocks, const int32_t* positions,
                                      const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size,
                                      int q_width, int nkv, int kd, int vd, int store, int* err, cudaStream_t stream) {
    if (T < 0 || q_width <= 0 || nkv <= 0 || kd <= 0 || vd <= 0 || !err || !positions || !req_of_token ||
        (store && (!pool || !block_table || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
#define QS_LAUNCH(TT) airun_launch(qkv_bias_store_kernel<TT>, dim3(T), dim3(256), 0, stream, proj, proj_stride, q_bias, k_bias, v_bias, \
        (TT*)q_out, (TT*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, q_width, nkv, kd, vd, store, err)
    if (dtype == AIRUN_DT_F32) QS_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) QS_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef QS_LAUNCH
    return airun_launch_status();
}

// One block per (token, query head).  Each warp walks every DA_WARPS-th visible key and keeps a running
// maximum, sum and value accumulator for each of the two maps; the warps' partial results are merged,
// the maps combined and the head normed at the end.  A token's result depends only on its own q,
// position and the keys it sees.
template <typename T>
__global__ __launch_bounds__(32 * DA_WARPS) void diff_attention_kernel(
    const T* __restrict__ q, T* __restrict__ out, long long out_stride, const T* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int nh, int nkv, int D, int Dv,
    float scale, float cap, int chunk, int window, float lambda, float eps, float out_scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* s_max = smem;                       // [2][DA_WARPS]
    float* s_sum = smem + 2 * DA_WARPS;        // [2][DA_WARPS]
    float* s_acc = smem + 4 * DA_WARPS;        // [2][DA_WARPS][Dv]
    const int t = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t], req = req_of_token[t];
    T* dst = out + (size_t)t * out_stride + (size_t)head * Dv;
    if (req < 0 || pos < 0 || req >= num_reqs) {      // a padding row
        if (req >= num_reqs && threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        for (int d = threadIdx.x; d < Dv; d += blockDim.x) dst[d] = from_f32<T>(0.0f);
        return;
    }
    const int kvh = head / (nh / nkv), kd = 2 * D;
    const T* qv = q + ((size_t)t * nh + head) * kd;
    float q1[DA_MAX_PER_LANE], q2[DA_MAX_PER_LANE], acc1[DA_MAX_PER_LANE], acc2[DA_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        q1[i] = d < D ? to_f32<T>(qv[d]) : 0.0f;
        q2[i] = d < D ? to_f32<T>(qv[D + d]) : 0.0f;
        acc1[i] = acc2[i] = 0.0f;
    }
    float max1 = -INFINITY, max2 = -INFINITY, sum1 = 0.0f, sum2 = 0.0f;
    const int32_t* bt = block_table + (size_t)req * max_blocks;
    int begin = chunk > 0 ? (pos / chunk) * chunk : 0;
    if (window > 0) begin = max(begin, pos - window + 1);
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    bool bad = false;
    const size_t page_elems = (size_t)nkv * page_size * (kd + Dv);
    for (int j = begin + warp; j <= pos; j += DA_WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const T* pk = pool + (size_t)page * page_elems;
        const T* kj = pk + ((size_t)kvh * page_size + (j - blk * page_size)) * kd;
        const T* vj = pk + (size_t)nkv * page_size * kd + ((size_t)kvh * page_size + (j - blk * page_size)) * Dv;
        float d1 = 0.0f, d2 = 0.0f;
#pragma unroll
        for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < D) {
                d1 = fmaf(q1[i], to_f32<T>(kj[d]), d1);
                d2 = fmaf(q2[i], to_f32<T>(kj[D + d]), d2);
            }
        }
        d1 = warp_sum(d1) * scale;
        d2 = warp_sum(d2) * scale;
        if (cap > 0.0f) { d1 = cap * tanhf(d1 * inv_cap); d2 = cap * tanhf(d2 * inv_cap); }
        const float n1 = fmaxf(max1, d1), n2 = fmaxf(max2, d2);
        const float c1 = expf(max1 - n1), c2 = expf(max2 - n2);     // exactly 0 on the first key
        const float p1 = expf(d1 - n1), p2 = expf(d2 - n2);
        sum1 = sum1 * c1 + p1;
        sum2 = sum2 * c2 + p2;
#pragma unroll
        for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < Dv) {
                const float vv = to_f32<T>(vj[d]);
                acc1[i] = fmaf(p1, vv, acc1[i] * c1);
                acc2[i] = fmaf(p2, vv, acc2[i] * c2);
            }
        }
        max1 = n1; max2 = n2;
    }
    if (bad && lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
    if (lane == 0) {
        s_max[warp] = max1; s_max[DA_WARPS + warp] = max2;
        s_sum[warp] = sum1; s_sum[DA_WARPS + warp] = sum2;
    }
#pragma unroll
    for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < Dv) {
            s_acc[(size_t)warp * Dv + d] = acc1[i];
            s_acc[(size_t)(DA_WARPS + warp) * Dv + d] = acc2[i];
        }
    }
    __syncthreads();
    if (warp != 0) return;
    float wgt[2][DA_WARPS], inv[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float gmax = -INFINITY, gsum = 0.0f;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) gmax = fmaxf(gmax, s_max[m * DA_WARPS + w]);
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) {
            wgt[m][w] = s_sum[m * DA_WARPS + w] > 0.0f ? expf(s_max[m * DA_WARPS + w] - gmax) : 0.0f;
            gsum += s_sum[m * DA_WARPS + w] * wgt[m][w];
        }
        inv[m] = gsum > 0.0f ? 1.0f / gsum : 0.0f;
    }
    float o[DA_MAX_PER_LANE], ss = 0.0f;
#pragma unroll
    for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        o[i] = 0.0f;
        if (d >= Dv) continue;
        float a1 = 0.0f, a2 = 0.0f;
#pragma unroll
        for (int w = 0; w < DA_WARPS; ++w) {
            a1 = fmaf(s_acc[(size_t)w * Dv + d], wgt[0][w], a1);
            a2 = fmaf(s_acc[(size_t)(DA_WARPS + w) * Dv + d], wgt[1][w], a2);
        }
        o[i] = a1 * inv[0] - lambda * (a2 * inv[1]);
        ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    const float nrm = out_scale / sqrtf(ss / (float)Dv + eps);
#pragma unroll
    for (int i = 0; i < DA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < Dv) dst[d] = from_f32<T>(o[i] * nrm);
    }
}

AIRUN_EXPORT int airun_diff_attention(const void* q, void* out, long long out_stride, const void* pool, int dtype,
                                      const int32_t* block_table, int max_blocks, const int32_t* positions,
                                      const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size,
                                      int nh, int nkv, int D, int Dv, float scale, float cap, int chunk, int window,
                                      float lambda, float eps, float out_scale, int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 32 * DA_MAX_PER_LANE || Dv <= 0 ||
        Dv > 32 * DA_MAX_PER_LANE || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || chunk < 0 || window < 0 ||
        !err || nh > 65535 || out_stride < (long long)nh * Dv)
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    dim3 grid(T, nh);
    const size_t smem = (size_t)(4 * DA_WARPS + 2 * DA_WARPS * Dv) * sizeof(float);
#define DA_LAUNCH(TT) airun_launch(diff_attention_kernel<TT>, grid, dim3(32 * DA_WARPS), smem, stream, (const TT*)q, (TT*)out, out_stride, \
        (const TT*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, nh, nkv, D, Dv, scale, cap, \
        chunk, window, lambda, eps, out_scale, err)
    if (dtype == AIRUN_DT_F32) DA_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) DA_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef DA_LAUNCH
    return airun_launch_status();
}
