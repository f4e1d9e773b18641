// Dense projections of one to four tokens as weight streams: y[t, n] = sum_k x[t, k] W[n, k].
//
// With so few tokens a projection is a read of its weights and nothing else, and what a step pays for is the
// number of launches between two layers.  The reference computes exactly this product one output at a time
// (tq_matmul, src/engine/tq_ops.c:270-343) and adds the bias, rotates and writes the cache afterwards
// (src/engine/tq_transformer.c:1044-1047, 1086-1093, 1343, 1371, 1452-1455).  Here:
//   tq_gemv            the product alone (the attention's output projection): float32 out
//   tq_qkv_gemv_rope   the fused query/key/value projection with everything that follows it in one launch: bias,
//                      rotary position encoding (half pairing, from the fp32 tables), queries to their buffer, keys
//                      and values straight into the cache pages; replaces a library GEMM and the
//                      qkv_rope_cache kernel for steps of up to four tokens
// A warp owns one output row (the fused form: the two rows of a rotation pair, d and d + head_dim / 2, of one head),
// its lanes cut K into 16-byte pieces and ask for all of them at once, before the kernel even waits for its
// predecessor; the tokens' rows sit in shared memory as bfloat16, sums are fp32, one shuffle reduction per output.  bfloat16 weights with K a multiple of 8; the Python side keeps the library
// product for everything else.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define GEMV_WARPS 8
#define GEMV_MAX_T 4
#define GEMV_KI 8                // 16-byte pieces of a row a lane has in flight per row (8 x 256 = 2,048 values of K)

__device__ __forceinline__ void gemv_widen(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint4 gemv_stream16(const void* p) {          // read once: do not keep it in the L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// A warp's NR weight rows against the T rows of x.  What bounds a product of this size is not bandwidth but the
// number of trips to memory one after another, so a lane asks for all its pieces of a row at once (GEMV_KI pieces
// per row: one trip for K up to 2,048, two up to 4,096), and the first trip starts BEFORE the kernel waits for the
// one ahead of it in the stream: weights do not depend on it.
template <int NR>
struct GemvRows {
    const __nv_bfloat16* w[NR];
    uint4 wv[NR][GEMV_KI];                                                // the pieces in flight (or just landed)
    __device__ __forceinline__ void ask(int K, int lane, int k0) {        // one trip: GEMV_KI pieces of every row
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int it = 0; it < GEMV_KI; ++it) {
                const int k = k0 + lane * 8 + it * 256;
                wv[r][it] = k < K ? gemv_stream16(w[r] + k) : make_uint4(0u, 0u, 0u, 0u);
            }
    }
    // after ask(K, lane, 0): the dots with the T rows of x in shared memory; every lane ends up with the full sums
    template <int T>
    __device__ __forceinline__ void dots(const __nv_bfloat16* __restrict__ s_x, int K, int lane, float (&acc)[NR][T]) {
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
        for (int k0 = 0; k0 < K; k0 += GEMV_KI * 256) {
            if (k0 != 0) ask(K, lane, k0);                                // the first trip was started by the caller
#pragma unroll
            for (int it = 0; it < GEMV_KI; ++it) {
                const int k = k0 + lane * 8 + it * 256;
                if (k < K) {
                    float xf[T][8];
#pragma unroll
                    for (int t = 0; t < T; ++t) gemv_widen(*reinterpret_cast<const uint4*>(s_x + (size_t)t * K + k), xf[t]);
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        float wf[8];
                        gemv_widen(wv[r][it], wf);
#pragma unroll
                        for (int t = 0; t < T; ++t)
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[r][t] = fmaf(wf[i], xf[t][i], acc[r][t]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t) acc[r][t] = tq_warp_sum(acc[r][t]);
    }
};

template <int T>
__device__ __forceinline__ void gemv_stage_x(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ s_x, int K) {
    tq_grid_wait();                    // x is what the previous kernel wrote; the weights were asked for before
    tq_grid_launch_dependents();
    const __nv_bfloat16* xs = tq_fresh(x);                 // loads of x stay behind the wait
    for (int i = threadIdx.x * 8; i < T * K; i += blockDim.x * 8)
        *reinterpret_cast<uint4*>(s_x + i) = *reinterpret_cast<const uint4*>(xs + i);
    __syncthreads();
}

// a warp per output row
template <int T>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float* __restrict__ y, int N, int K) {
    extern __shared__ __align__(16) __nv_bfloat16 s_gemv_x[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * GEMV_WARPS + warp;
    GemvRows<1> rows;
    rows.w[0] = w + (size_t)min(n, N - 1) * K;
    rows.ask(K, lane, 0);
    gemv_stage_x<T>(x, s_gemv_x, K);
    float acc[1][T];
    rows.template dots<T>(s_gemv_x, K, lane, acc);
    if (lane == 0 && n < N) {
#pragma unroll
        for (int t = 0; t < T; ++t) y[(size_t)t * N + n] = acc[0][t];
    }
}

// x [T, K] bf16, w [N, K] bf16, y [T, N] float32; 1 <= T <= 4, K % 8 == 0, 16-byte aligned operands.
TQ_EXPORT int tq_gemv(const void* x, const void* w, float* y, int T_, int N, int K, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ >= 1 && T_ <= GEMV_MAX_T, "gemv: %d tokens; this kernel takes 1 to %d", T_, GEMV_MAX_T);
    TQ_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemv: bad sizes N=%d K=%d (K must be a multiple of 8)", N, K);
    TQ_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemv: operands must be 16-byte aligned");
    const size_t smem = (size_t)T_ * K * sizeof(__nv_bfloat16);
    TQ_REQUIRE(smem <= 48 * 1024, "gemv: %d rows of %d values do not fit 48 KiB of shared memory", T_, K);
    const int grid = (N + GEMV_WARPS - 1) / GEMV_WARPS;
#define GEMV_CASE(TT) case TT: tq_launch(grid, GEMV_WARPS * 32, smem, stream)(gemv_kernel<TT>, (const __nv_bfloat16*)x, \
                                         (const __nv_bfloat16*)w, y, N, K); break;
    switch (T_) { GEMV_CASE(1) GEMV_CASE(2) GEMV_CASE(3) GEMV_CASE(4) }
#undef GEMV_CASE
    TQ_CHECK_LAUNCH("gemv");
    return 0;
}

// ---------------------------------------------------------------------------------------
// The fused projection of queries, keys and values.  Weight rows: [nh heads of queries, nkv of keys, nkv of values]
// x head_dim.  A warp takes rotation pairs (rows d and d + hd/2 of one head), two pairs at a time.
// ---------------------------------------------------------------------------------------
template <int T, typename TB>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
qkv_gemv_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const TB* __restrict__ bias,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions,
                     const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int table_stride,
                     int page_size, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ cache, int write_kv,
                     int K, int nh, int nkv, int hd, int n_seqs, int n_pages) {
    extern __shared__ __align__(16) __nv_bfloat16 s_gemv_x[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = hd >> 1;
    const int heads = write_kv ? nh + 2 * nkv : nh;
    const int pairs = heads * half;
    const int p = min((int)blockIdx.x * GEMV_WARPS + warp, pairs - 1);   // a warp per rotation pair
    const bool mine = (int)blockIdx.x * GEMV_WARPS + warp < pairs;
    const int h = p / half, i = p - h * half;
    GemvRows<2> rows;
    rows.w[0] = w + ((size_t)h * hd + i) * K;
    rows.w[1] = w + ((size_t)h * hd + half + i) * K;
    rows.ask(K, lane, 0);
    gemv_stage_x<T>(x, s_gemv_x, K);
    float acc[2][T];
    rows.template dots<T>(s_gemv_x, K, lane, acc);
    if (lane < T && mine) {                                              // lane t finishes the pair for token t
        float a = 0.f, c = 0.f;
#pragma unroll
        for (int tt = 0; tt < T; ++tt)
            if (tt == lane) { a = acc[0][tt]; c = acc[1][tt]; }
        const int t = lane;
        // the library product this replaces hands bfloat16 to the rotation: the same rounding here
        a = __bfloat162float(__float2bfloat16_rn(a));
        c = __bfloat162float(__float2bfloat16_rn(c));
        if (bias) { a += tq_to_float(bias[(size_t)h * hd + i]); c += tq_to_float(bias[(size_t)h * hd + half + i]); }
        const int pos = positions[t];
        const bool is_v = h >= nh + nkv;
        if (!is_v && cos_t) {
            const float cs = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
            const float ra = a * cs - c * sn, rc = a * sn + c * cs;
            a = ra; c = rc;
        }
        __nv_bfloat16* dst;
        if (h < nh) {
            dst = q_out + ((size_t)t * nh + h) * hd;
        } else {
            const int page = TQ_CHECKED(page_table[(size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride
                                                   + TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)],
                                        n_pages, TQ_IDX_PAGE);
            const int kvh = is_v ? h - nh - nkv : h - nh;
            dst = cache + (size_t)page * 2 * nkv * page_size * hd + (size_t)(pos % page_size) * hd
                  + ((size_t)(is_v ? 1 : 0) * nkv + kvh) * page_size * hd;
        }
        dst[i] = __float2bfloat16_rn(a);
        dst[half + i] = __float2bfloat16_rn(c);
    }
}

// x [T, K] bf16 (the normed rows); w [(nh + 2 nkv) * hd, K] bf16; bias of that many values or null (bf16 or fp32);
// cos/sin [positions, hd / 2] fp32 or both null; q_out [T, nh, hd] bf16; cache [pages, 2, nkv, page_size, hd] bf16
// (write_kv = 0: only the queries are produced).  1 <= T <= 4, K % 8 == 0, hd even.
TQ_EXPORT int tq_qkv_gemv_rope(const void* x, const void* w, const void* bias, int bias_dtype, const float* cos_t,
                               const float* sin_t, const int* positions, const int* seq_of_token, const int* page_table,
                               int table_stride, int page_size, void* q_out, void* cache, int write_kv, int T_, int K,
                               int nh, int nkv, int hd, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ >= 1 && T_ <= GEMV_MAX_T, "qkv_gemv_rope: %d tokens; this kernel takes 1 to %d", T_, GEMV_MAX_T);
    TQ_REQUIRE(K > 0 && K % 8 == 0 && hd >= 2 && hd % 2 == 0, "qkv_gemv_rope: bad sizes K=%d head size %d", K, hd);
    TQ_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qkv_gemv_rope: cos and sin tables must come together");
    TQ_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "qkv_gemv_rope: operands must be 16-byte aligned");
    const size_t smem = (size_t)T_ * K * sizeof(__nv_bfloat16);
    TQ_REQUIRE(smem <= 48 * 1024, "qkv_gemv_rope: %d rows of %d values do not fit 48 KiB of shared memory", T_, K);
    const int pairs = (write_kv ? nh + 2 * nkv : nh) * (hd / 2);
    const int grid = (pairs + GEMV_WARPS - 1) / GEMV_WARPS;
#define QKV_CASE(TT)                                                                                            \
    case TT: TQ_DISPATCH(bias ? bias_dtype : TQ_BF16, TB,                                                       \
        (tq_launch(grid, GEMV_WARPS * 32, smem, stream)(qkv_gemv_rope_kernel<TT, TB>, (const __nv_bfloat16*)x,  \
            (const __nv_bfloat16*)w, (const TB*)bias, cos_t, sin_t, positions, seq_of_token, page_table, table_stride, \
            page_size, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, write_kv, K, nh, nkv, hd, n_seqs, n_pages))); break;
    switch (T_) { QKV_CASE(1) QKV_CASE(2) QKV_CASE(3) QKV_CASE(4) }
#undef QKV_CASE
    TQ_CHECK_LAUNCH("qkv_gemv_rope");
    return 0;
}
