// Attention over the paged key/value cache: the exact (any size) kernels.
//
//   tq_qkv_rope_cache  bias + rotary position encoding on the fused QKV projection; queries go to
//                      a buffer, keys and values straight into the cache pages
//   tq_attention       softmax(q.K/sqrt(hd)) V for every (token, head) over the cache, causal,
//                      with an optional window; one code path for prompts and for decoding
//
// Formulas as the reference computes them on the CPU (src/engine/tq_transformer.c):
//   bias after the projection :1044-1047, 1086-1093; rotary src/engine/tq_ops.c:1418-1448
//   (pairs (2i, 2i+1) there; pairing 0 here is the checkpoint layout (i, i+hd/2));
//   cache write at the token's position :1371, 1452-1455; head h reads KV head h/(nh/nkv) :1679;
//   score = q.k/sqrt(hd) :1633, 1909-1936; window start :1646-1654; softmax :1960; PV :2183-2191.
// Scores, softmax and the weighted sum are fp32 on both paths; rotation angles come from an fp32
// table indexed by position.
//
// Cache layout of one layer: [page][2 (K,V)][kv head][slot in page][head dim]; a sequence's
// position p lives in page table[seq][p / page_size] at slot p % page_size.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define TQ_MAX_HEAD_DIM 256

// ---------------------------------------------------------------------------------------
// grid (T, nh + 2*nkv) [or (T, nh) when keys/values are not written]; one pair per thread
// ---------------------------------------------------------------------------------------
template <typename TA, typename TB>
__global__ void qkv_rope_cache_kernel(const TA* __restrict__ qkv, const TB* __restrict__ bias,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      int pairing, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ page_table,
                                      int table_stride, int page_size, TA* __restrict__ q_out,
                                      TA* __restrict__ cache, int nh, int nkv, int hd) {
    const int t = blockIdx.x, j = blockIdx.y, i = threadIdx.x;
    const int half = hd >> 1;
    if (i >= half) return;
    const int width = (nh + 2 * nkv) * hd;
    const TA* src = qkv + (size_t)t * width + (size_t)j * hd;
    const TB* b = bias ? bias + (size_t)j * hd : nullptr;
    const int pos = positions[t];
    int ia, ib;
    if (pairing == 0) { ia = i; ib = i + half; } else { ia = 2 * i; ib = 2 * i + 1; }
    float a = tq_to_float(src[ia]), c = tq_to_float(src[ib]);
    if (b) { a += tq_to_float(b[ia]); c += tq_to_float(b[ib]); }
    const bool is_v = j >= nh + nkv;
    if (!is_v && cos_t) {
        const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
        const float ra = a * cs - c * sn, rc = a * sn + c * cs;
        a = ra; c = rc;
    }
    TA* dst;
    if (j < nh) {
        dst = q_out + ((size_t)t * nh + j) * hd;
    } else {
        const int kvh = is_v ? j - nh - nkv : j - nh;
        const int page = page_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
        dst = cache + ((((size_t)page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + pos % page_size) * hd;
    }
    dst[ia] = tq_from_float<TA>(a);
    dst[ib] = tq_from_float<TA>(c);
}

TQ_EXPORT int tq_qkv_rope_cache(const void* qkv, int act_dtype, const void* bias, int bias_dtype,
                                const float* cos_t, const float* sin_t, int pairing,
                                const int* positions, const int* seq_of_token, const int* page_table,
                                int table_stride, int page_size, void* q_out, void* cache, int write_kv,
                                int T_, int nh, int nkv, int hd, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd % 2 == 0 && hd >= 2 && hd <= 2048, "qkv_rope_cache: head size %d must be even and <= 2048", hd);
    TQ_REQUIRE(pairing == 0 || pairing == 1, "qkv_rope_cache: pairing %d is neither half (0) nor interleaved (1)", pairing);
    TQ_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qkv_rope_cache: cos and sin tables must come together");
    const int heads = write_kv ? nh + 2 * nkv : nh;
    TQ_REQUIRE(heads <= 65535, "qkv_rope_cache: %d heads exceed the grid limit", heads);
    dim3 grid(T_, heads);
    const int threads = ((hd / 2 + 31) / 32) * 32;
    TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(bias_dtype, TB,
        (qkv_rope_cache_kernel<TA, TB><<<grid, threads, 0, stream>>>(
            (const TA*)qkv, (const TB*)bias, cos_t, sin_t, pairing, positions, seq_of_token, page_table,
            table_stride, page_size, (TA*)q_out, (TA*)cache, nh, nkv, hd))));
    TQ_CHECK_LAUNCH("qkv_rope_cache");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Exact attention: grid (T, nh), 4 warps per block.  Warp w takes keys start+w, start+w+4, …;
// a lane holds head elements lane, lane+32, …; online softmax per warp, merged through shared
// memory.  The order of the sums depends only on (start, pos), never on the batch.
// ---------------------------------------------------------------------------------------
#define ATT_WARPS 4
#define ATT_EPL (TQ_MAX_HEAD_DIM / 32)   // head elements per lane

template <typename TA>
__global__ void attention_kernel(const TA* __restrict__ q, const TA* __restrict__ cache,
                                 const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ page_table, int table_stride, int page_size,
                                 int window, float scale, TA* __restrict__ out, int nh, int nkv, int hd) {
    __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
    __shared__ float s_acc[ATT_WARPS][TQ_MAX_HEAD_DIM];
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = h / (nh / nkv);
    const int pos = positions[t];
    const int start = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = page_table + (size_t)seq_of_token[t] * table_stride;

    float qv[ATT_EPL], acc[ATT_EPL];
    const TA* qp = q + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int j = 0; j < ATT_EPL; ++j) {
        const int e = lane + 32 * j;
        qv[j] = e < hd ? tq_to_float(qp[e]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int p = start + warp; p <= pos; p += ATT_WARPS) {
        const int page = table[p / page_size];
        const TA* kp = cache + ((((size_t)page * 2 + 0) * nkv + g) * page_size + p % page_size) * hd;
        const TA* vp = kp + (size_t)nkv * page_size * hd;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < ATT_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < hd) s += qv[j] * tq_to_float(kp[e]);
        }
        s = tq_warp_sum(s) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);          // exp(-inf) = 0 on the first key
        const float pexp = expf(s - m_new);
        l = l * corr + pexp;
#pragma unroll
        for (int j = 0; j < ATT_EPL; ++j) {
            const int e = lane + 32 * j;
            if (e < hd) acc[j] = acc[j] * corr + pexp * tq_to_float(vp[e]);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < ATT_EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < hd) s_acc[warp][e] = acc[j];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f;
    float f[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);
        L += s_l[w] * f[w];
    }
    TA* op = out + ((size_t)t * nh + h) * hd;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) v += s_acc[w][e] * f[w];
        op[e] = tq_from_float<TA>(v / L);
    }
}

TQ_EXPORT int tq_attention(const void* q, const void* cache, int act_dtype, const int* positions,
                           const int* seq_of_token, const int* page_table, int table_stride, int page_size,
                           int window, float scale, void* out, int T_, int nh, int nkv, int hd,
                           cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd >= 1 && hd <= TQ_MAX_HEAD_DIM, "attention: head size %d exceeds %d", hd, TQ_MAX_HEAD_DIM);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "attention: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(nh <= 65535, "attention: %d heads exceed the grid limit", nh);
    TQ_REQUIRE(window >= 0, "attention: negative window %d", window);
    dim3 grid(T_, nh);
    TQ_DISPATCH(act_dtype, TA,
        (attention_kernel<TA><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const TA*)q, (const TA*)cache, positions, seq_of_token, page_table, table_stride, page_size,
            window, scale, (TA*)out, nh, nkv, hd)));
    TQ_CHECK_LAUNCH("attention");
    return 0;
}
