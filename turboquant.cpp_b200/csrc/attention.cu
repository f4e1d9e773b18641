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

// eight consecutive elements: fetched raw (so that the next group's loads can be in flight while the
// current group is computed), widened to fp32 when used
template <typename T> struct Vec8 { };
template <> struct Vec8<__nv_bfloat16> {
    struct Raw { uint4 v; };
    static __device__ __forceinline__ Raw fetch(const __nv_bfloat16* p) { Raw r; r.v = *reinterpret_cast<const uint4*>(p); return r; }
    static __device__ __forceinline__ void widen(const Raw& r, float (&f)[8]) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) { widen(fetch(p), f); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint4 v;
        uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); u[i] = *reinterpret_cast<const uint32_t*>(&h); }
        *reinterpret_cast<uint4*>(p) = v;
    }
};
template <> struct Vec8<float> {
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw fetch(const float* p) {
        Raw r; r.a = *reinterpret_cast<const float4*>(p); r.b = *reinterpret_cast<const float4*>(p + 4); return r;
    }
    static __device__ __forceinline__ void widen(const Raw& r, float (&f)[8]) {
        f[0] = r.a.x; f[1] = r.a.y; f[2] = r.a.z; f[3] = r.a.w; f[4] = r.b.x; f[5] = r.b.y; f[6] = r.b.z; f[7] = r.b.w;
    }
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) { widen(fetch(p), f); }
    static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// ---------------------------------------------------------------------------------------
// A block walks (head, pair) indices of one token's fused QKV row; with few tokens several blocks share a row.
// ---------------------------------------------------------------------------------------
template <typename TA, typename TB>
__global__ void qkv_rope_cache_kernel(const TA* __restrict__ qkv, const TB* __restrict__ bias,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      int pairing, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ page_table,
                                      int table_stride, int page_size, TA* __restrict__ q_out,
                                      TA* __restrict__ cache, int heads, int nh, int nkv, int hd, int vec8,
                                      int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int width = (nh + 2 * nkv) * hd;
    const TA* row = qkv + (size_t)t * width;
    const int pos = positions[t];
    const float* cs_row = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn_row = sin_t ? sin_t + (size_t)pos * half : nullptr;
    size_t page_base = 0;
    if (heads > nh) {
        const int page = TQ_CHECKED(page_table[(size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride
                                               + TQ_CHECKED(pos / page_size, table_stride, TQ_IDX_TABLE_COLUMN)],
                                    n_pages, TQ_IDX_PAGE);
        page_base = (size_t)page * 2 * nkv * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    if (vec8) {
        // half pairing, head size a multiple of 16, 16-byte aligned rows: a thread takes eight pairs,
        // elements i..i+7 of the first half of a head and the same of the second half
        const int groups = half >> 3;
        for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < heads * groups; idx += gridDim.y * blockDim.x) {
            const int j = idx / groups, i = (idx - j * groups) * 8;
            const TA* src = row + (size_t)j * hd;
            float a[8], c[8];
            Vec8<TA>::load(src + i, a);
            Vec8<TA>::load(src + half + i, c);
            if (bias) {
                float ba[8], bc[8];
                Vec8<TB>::load(bias + (size_t)j * hd + i, ba);
                Vec8<TB>::load(bias + (size_t)j * hd + half + i, bc);
#pragma unroll
                for (int e = 0; e < 8; ++e) { a[e] += ba[e]; c[e] += bc[e]; }
            }
            const bool is_v = j >= nh + nkv;
            if (!is_v && cs_row) {
                float cs[8], sn[8];                        // i is a multiple of 8 and a table row of 4 floats: 16-byte loads
                Vec8<float>::load(cs_row + i, cs);
                Vec8<float>::load(sn_row + i, sn);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float ra = a[e] * cs[e] - c[e] * sn[e], rc = a[e] * sn[e] + c[e] * cs[e];
                    a[e] = ra; c[e] = rc;
                }
            }
            TA* dst;
            if (j < nh) {
                dst = q_out + ((size_t)t * nh + j) * hd;
            } else {
                const int kvh = is_v ? j - nh - nkv : j - nh;
                dst = cache + page_base + ((size_t)(is_v ? 1 : 0) * nkv + kvh) * page_size * hd;
            }
            Vec8<TA>::store(dst + i, a);
            Vec8<TA>::store(dst + half + i, c);
        }
        return;
    }
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < heads * half; idx += gridDim.y * blockDim.x) {
        const int j = idx / half, i = idx - j * half;
        const TA* src = row + (size_t)j * hd;
        int ia, ib;
        if (pairing == 0) { ia = i; ib = i + half; } else { ia = 2 * i; ib = 2 * i + 1; }
        float a = tq_to_float(src[ia]), c = tq_to_float(src[ib]);
        if (bias) { a += tq_to_float(bias[(size_t)j * hd + ia]); c += tq_to_float(bias[(size_t)j * hd + ib]); }
        const bool is_v = j >= nh + nkv;
        if (!is_v && cs_row) {
            const float cs = cs_row[i], sn = sn_row[i];
            const float ra = a * cs - c * sn, rc = a * sn + c * cs;
            a = ra; c = rc;
        }
        TA* dst;
        if (j < nh) {
            dst = q_out + ((size_t)t * nh + j) * hd;
        } else {
            const int kvh = is_v ? j - nh - nkv : j - nh;
            dst = cache + page_base + ((size_t)(is_v ? 1 : 0) * nkv + kvh) * page_size * hd;
        }
        dst[ia] = tq_from_float<TA>(a);
        dst[ib] = tq_from_float<TA>(c);
    }
}

TQ_EXPORT int tq_qkv_rope_cache(const void* qkv, int act_dtype, const void* bias, int bias_dtype,
                                const float* cos_t, const float* sin_t, int pairing,
                                const int* positions, const int* seq_of_token, const int* page_table,
                                int table_stride, int page_size, void* q_out, void* cache, int write_kv,
                                int T_, int nh, int nkv, int hd, int n_seqs, int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd % 2 == 0 && hd >= 2 && hd <= 2048, "qkv_rope_cache: head size %d must be even and <= 2048", hd);
    TQ_REQUIRE(pairing == 0 || pairing == 1, "qkv_rope_cache: pairing %d is neither half (0) nor interleaved (1)", pairing);
    TQ_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qkv_rope_cache: cos and sin tables must come together");
    const int heads = write_kv ? nh + 2 * nkv : nh;
    const int esize = act_dtype == TQ_F32 ? 4 : 2;
    const int vec8 = pairing == 0 && hd % 16 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)q_out % 16) == 0 &&
                     ((uintptr_t)cache % 16) == 0 && ((size_t)hd * esize) % 16 == 0 &&
                     ((uintptr_t)cos_t % 16) == 0 && ((uintptr_t)sin_t % 16) == 0 &&
                     ((uintptr_t)bias % 16) == 0 && ((size_t)hd * (bias_dtype == TQ_F32 ? 4 : 2)) % 16 == 0;
    const int pairs = vec8 ? heads * (hd / 16) : heads * (hd / 2);      // work items per token
    // long steps: one block per token whose threads cover the token's work items in whole rounds
    const int threads = T_ >= 512 ? (pairs % 192 == 0 ? 192 : (pairs % 128 == 0 ? 128 : 256))
                                  : (pairs >= 1024 ? 256 : (pairs >= 256 ? 128 : 64));
    // few tokens: several blocks share a token's row, so that the step still fills the GPU
    int chunks = T_ >= 512 ? 1 : (pairs + threads - 1) / threads;
    if (chunks > 64) chunks = 64;
    TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(bias_dtype, TB,
        (tq_launch(dim3(T_, chunks), threads, 0, stream)(qkv_rope_cache_kernel<TA, TB>, 
            (const TA*)qkv, (const TB*)bias, cos_t, sin_t, pairing, positions, seq_of_token, page_table,
            table_stride, page_size, (TA*)q_out, (TA*)cache, heads, nh, nkv, hd, vec8, n_seqs, n_pages))));
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
                                 int window, float scale, TA* __restrict__ out, int nh, int nkv, int hd,
                                 int n_seqs, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
    __shared__ float s_acc[ATT_WARPS][TQ_MAX_HEAD_DIM];
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = h / (nh / nkv);
    const int pos = positions[t];
    const int start = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;

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
        const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
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
                           int window, float scale, void* out, int T_, int nh, int nkv, int hd, int n_seqs, int n_pages,
                           cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd >= 1 && hd <= TQ_MAX_HEAD_DIM, "attention: head size %d exceeds %d", hd, TQ_MAX_HEAD_DIM);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "attention: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(nh <= 65535, "attention: %d heads exceed the grid limit", nh);
    TQ_REQUIRE(window >= 0, "attention: negative window %d", window);
    dim3 grid(T_, nh);
    TQ_DISPATCH(act_dtype, TA,
        (tq_launch(grid, ATT_WARPS * 32, 0, stream)(attention_kernel<TA>, 
            (const TA*)q, (const TA*)cache, positions, seq_of_token, page_table, table_stride, page_size,
            window, scale, (TA*)out, nh, nkv, hd, n_seqs, n_pages)));
    TQ_CHECK_LAUNCH("attention");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Split attention for decoding (and any step with few tokens per sequence): the keys of one
// (token, KV head) are cut into `n_splits` ranges, one CTA per range; the CTA that finishes last
// (found by a ticket counter, without waiting) merges the ranges' partial softmax states in range order.  A key row is read by LPK = hd/8 lanes with one 16-byte load
// each (two for fp32), so a warp covers 32/LPK keys per instruction and eight keys per iteration
// with all loads in flight together; the G query heads that share the KV head are computed from
// the same registers.  Partial state per (token, head, split): max, sum, hd weighted values (fp32).
// STAGES > 0 (bfloat16, one query head per KV head, head size 128): the loads are 16-byte cp.async
// copies into a ring in shared memory, STAGES - 1 groups ahead of the one being computed, every lane
// copying and reading back only its own 16 bytes (no barrier between the warps).  The arithmetic and its
// order are the same, so both forms give the same bits.  With two stages the kernel needs 48 registers
// instead of 113 and 36 KiB of shared memory: six CTAs per SM instead of four.  Measured on B200 at 16
// heads x 128 and 2,048 keys: 64 tokens (4,096 CTAs) 170 us against 180 us; 8 tokens (512 CTAs, less than
// one wave either way) 28 us against 29 us alone but 2 us per layer slower inside a decode step.  So the
// ring serves launches of more than two waves of the register form, and the registers the others.
// ---------------------------------------------------------------------------------------
#define SPLIT_WARPS 4
#define SPLIT_REGISTER_CTAS_PER_SM 4     // CTAs of the register form an SM runs at once

__device__ __forceinline__ void split_copy16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void split_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void split_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// bytes of the ring: warps x stages x (K and V loads of a group) x 32 lanes x 16 bytes
template <typename TA, int LPK, int STAGES> constexpr int split_ring_bytes() {
    constexpr int KPI = 32 / LPK, GS = KPI > 8 ? KPI : 8, LOADS = GS / KPI;
    return SPLIT_WARPS * STAGES * 2 * LOADS * 32 * 16;
}

// stages of the ring for an element type and head size (0: this shape has no ring form)
template <typename TA, int LPK> constexpr int split_stages() { return sizeof(TA) == 2 && LPK == 16 ? 2 : 0; }

// The CTA that finishes last among the n_splits of a (token, KV head) merges their partial states, in the order of
// the ranges whichever CTA it is.  Nobody waits: each CTA publishes its state, takes a ticket and leaves unless the
// ticket is the last one.  Kept out of line: the split kernel's loop should not pay registers for it.
// rows: the first of this CTA's G heads in `partial` ([head][split][HD + 2]); out_rows: the same heads in `out`.
template <typename TA, int HD>
__device__ __noinline__ void split_merge_by_last(const float* __restrict__ partial, int n_splits, int* __restrict__ ticket,
                                                 TA* __restrict__ out_rows, const float* __restrict__ rows, int G) {
    __shared__ int s_last;
    __threadfence();                              // this thread's part of the state is visible before the ticket is taken
    __syncthreads();
    if (threadIdx.x == 0) {
        const int n = atomicAdd(ticket, 1);
        s_last = n == n_splits - 1;
        if (s_last) *ticket = 0;                  // every ticket of this launch has been taken: ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();                              // the others' states, published before their tickets, are visible now
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int h = idx / HD, d = idx % HD;
        const float* p = rows + (size_t)h * n_splits * (HD + 2);
        float M = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, __ldcg(p + (size_t)sp * (HD + 2)));
        float L = 0.f, a = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const float ms = __ldcg(p + (size_t)sp * (HD + 2));
            if (ms != -INFINITY) {
                const float f = expf(ms - M);
                L += __ldcg(p + (size_t)sp * (HD + 2) + 1) * f;
                a += __ldcg(p + (size_t)sp * (HD + 2) + 2 + d) * f;
            }
        }
        out_rows[(size_t)h * HD + d] = tq_from_float<TA>(a / L);
    }
}

template <typename TA, int LPK, int GC, int STAGES>
__global__ void __launch_bounds__(SPLIT_WARPS * 32)
attention_split_kernel(const TA* __restrict__ q, const TA* __restrict__ cache, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int table_stride,
                       int page_size, int window, float scale, float* __restrict__ partial, int n_splits,
                       int* __restrict__ arrived, TA* __restrict__ out, int nh, int nkv, int n_seqs, int n_pages,
                       int early_keys) {
    // early_keys: a decode step, in which the kernel ahead of this one wrote one thing into the cache, the keys and
    // values at each token's own position (and the queries); positions, page table and every older key were there
    // before that kernel started.  A warp whose first group of keys lies wholly below its token's position asks for
    // that group before it waits for the kernel ahead: the first round trip to DRAM overlaps that kernel's end.
    if (!early_keys) {
        tq_grid_wait();                    // everything below may read what the previous kernel wrote
        tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    }
    constexpr int HD = LPK * 8;
    constexpr int KPI = 32 / LPK;            // keys per load instruction of a warp
    constexpr int GS = KPI > 8 ? KPI : 8;    // keys per iteration of a warp (a group of absolute positions)
    constexpr int LOADS = GS / KPI;          // load instructions per iteration
    constexpr int NSTATE = SPLIT_WARPS * KPI; // partial states to merge inside the CTA
    __shared__ float s_m[NSTATE][GC], s_l[NSTATE][GC];
    __shared__ float s_acc[NSTATE][GC][HD];
    // more query heads per KV head than a CTA keeps in registers (GC): the heads are shared out over `chunks` CTAs
    // that sit side by side in the grid, so the second reads from the L2 what the first brought in
    const int G_all = nh / nkv;
    const int chunks = (G_all + GC - 1) / GC;
    const int t = blockIdx.x / chunks, chunk = blockIdx.x - t * chunks, g = blockIdx.y, split = blockIdx.z;
    const int h0 = chunk * GC;                           // first of this CTA's heads within the KV head's group
    const int G = min(GC, G_all - h0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LPK, part = lane / LPK;       // part: which of the KPI keys of a load
    const int pos = positions[t];
    const int start = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
    // this split's keys: whole groups of GS absolute positions
    const int first8 = start / GS, last8 = pos / GS;                   // inclusive groups
    const int groups = last8 - first8 + 1;
    const int per = (groups + n_splits - 1) / n_splits;
    const int gb = first8 + split * per, ge = min(last8 + 1, gb + per);

    using Raw = typename Vec8<TA>::Raw;
    static_assert(STAGES == 0 || sizeof(Raw) == 16, "the ring holds 16-byte loads");
    // the cache and the queries as the code below reads them: renewed behind a wait that comes late (tq_fresh), so
    // that no load of what the kernel ahead wrote is moved in front of that wait
    const TA* kv = cache;
    const TA* qs = q;
    // the keys and values of a group of GS positions, as this lane reads them
    auto fetch_group = [&](int grp, Raw (&kr)[LOADS], Raw (&vr)[LOADS]) {
        const int p0 = grp * GS;
        const int page = TQ_CHECKED(table[TQ_CHECKED(p0 / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const TA* kbase = kv + (((size_t)page * 2 + 0) * nkv + g) * page_size * HD + (size_t)(p0 % page_size) * HD;
        const TA* vbase = kbase + (size_t)nkv * page_size * HD;
#pragma unroll
        for (int j = 0; j < LOADS; ++j) kr[j] = Vec8<TA>::fetch(kbase + (size_t)(j * KPI + part) * HD + sub * 8);
#pragma unroll
        for (int j = 0; j < LOADS; ++j) vr[j] = Vec8<TA>::fetch(vbase + (size_t)(j * KPI + part) * HD + sub * 8);
    };
    Raw kr[LOADS], vr[LOADS];
    // the ring: [warp][stage][K loads, then V loads][lane] of 16 bytes, a lane's own slots only
    extern __shared__ __align__(16) unsigned char s_split_ring[];
    Raw* ring = reinterpret_cast<Raw*>(s_split_ring) + (size_t)warp * (STAGES > 0 ? STAGES : 1) * 2 * LOADS * 32 + lane;
    auto copy_group = [&](int grp, int stage) {
        const int p0 = grp * GS;
        const int page = TQ_CHECKED(table[TQ_CHECKED(p0 / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const TA* kbase = kv + (((size_t)page * 2 + 0) * nkv + g) * page_size * HD + (size_t)(p0 % page_size) * HD;
        const TA* vbase = kbase + (size_t)nkv * page_size * HD;
        Raw* dst = ring + (size_t)stage * 2 * LOADS * 32;
#pragma unroll
        for (int j = 0; j < LOADS; ++j) split_copy16(dst + j * 32, kbase + (size_t)(j * KPI + part) * HD + sub * 8);
#pragma unroll
        for (int j = 0; j < LOADS; ++j) split_copy16(dst + (LOADS + j) * 32, vbase + (size_t)(j * KPI + part) * HD + sub * 8);
    };
    int next_grp = gb + warp, next_stage = 0, stage = 0;     // ring: the next group to copy and where; the stage to read
    // the groups asked for ahead of the loop (one, or STAGES - 1 of the ring) end below the token's own position?
    const bool keys_ahead = early_keys && (gb + warp + (STAGES > 1 ? STAGES - 2 : 0) * SPLIT_WARPS) * GS + GS - 1 < pos;
    if (early_keys && !keys_ahead) { tq_grid_wait(); tq_grid_launch_dependents(); kv = tq_fresh(kv); }
    if (STAGES > 0) {
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) {                // one commit per group, also past the end: the count is uniform
            if (next_grp < ge) copy_group(next_grp, next_stage);
            split_commit();
            next_grp += SPLIT_WARPS;
            next_stage = next_stage + 1 == STAGES ? 0 : next_stage + 1;
        }
    } else if (gb + warp < ge) fetch_group(gb + warp, kr, vr);
    if (keys_ahead) { tq_grid_wait(); tq_grid_launch_dependents(); kv = tq_fresh(kv); }
    if (early_keys) qs = tq_fresh(qs);
    float qv[GC][8], acc[GC][8], m[GC], l[GC];
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h < G) Vec8<TA>::load(qs + ((size_t)t * nh + (size_t)g * G_all + h0 + h) * HD + sub * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { qv[h][i] = f[i] * scale; acc[h][i] = 0.f; }
    }
    for (int grp = gb + warp; grp < ge; grp += SPLIT_WARPS) {
        const int p0 = grp * GS;
        float kf[LOADS][8], vf[LOADS][8];
        if (STAGES > 0) {
            // the slot filled now was read one iteration ago, and what was read there has been used since
            if (next_grp < ge) copy_group(next_grp, next_stage);
            split_commit();
            next_grp += SPLIT_WARPS;
            next_stage = next_stage + 1 == STAGES ? 0 : next_stage + 1;
            split_wait<(STAGES > 0 ? STAGES - 1 : 0)>();      // all but the newest STAGES - 1 groups have landed: this one has
            const Raw* src = ring + (size_t)stage * 2 * LOADS * 32;
#pragma unroll
            for (int j = 0; j < LOADS; ++j) { kr[j] = src[j * 32]; vr[j] = src[(LOADS + j) * 32]; }
            stage = stage + 1 == STAGES ? 0 : stage + 1;
        }
#pragma unroll
        for (int j = 0; j < LOADS; ++j) { Vec8<TA>::widen(kr[j], kf[j]); Vec8<TA>::widen(vr[j], vf[j]); }
        if (STAGES == 0 && grp + SPLIT_WARPS < ge) fetch_group(grp + SPLIT_WARPS, kr, vr);      // next group's loads fly during this one's math
        float s[LOADS][GC];
#pragma unroll
        for (int j = 0; j < LOADS; ++j)
#pragma unroll
            for (int h = 0; h < GC; ++h) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(qv[h][i], kf[j][i], d);
                s[j][h] = d;
            }
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < LOADS; ++j)
#pragma unroll
                for (int h = 0; h < GC; ++h) s[j][h] += __shfl_xor_sync(0xffffffffu, s[j][h], o);
#pragma unroll
        for (int h = 0; h < GC; ++h) {
            float mx = m[h];
#pragma unroll
            for (int j = 0; j < LOADS; ++j) {
                const int p = p0 + j * KPI + part;
                if (p < start || p > pos) s[j][h] = -INFINITY;
                mx = fmaxf(mx, s[j][h]);
            }
            if (mx == -INFINITY) continue;                 // nothing visible yet for this lane group
            const float corr = expf(m[h] - mx);
            float lsum = l[h] * corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][i] *= corr;
#pragma unroll
            for (int j = 0; j < LOADS; ++j) {
                const float pe = expf(s[j][h] - mx);       // exp(-inf) = 0 for masked keys
                lsum += pe;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(pe, vf[j][i], acc[h][i]);
            }
            m[h] = mx; l[h] = lsum;
        }
    }
    // merge the CTA's NSTATE partial states
    const int st = warp * KPI + part;
#pragma unroll
    for (int h = 0; h < GC; ++h) {
        if (sub == 0) { s_m[st][h] = m[h]; s_l[st][h] = l[h]; }
#pragma unroll
        for (int i = 0; i < 8; ++i) s_acc[st][h][sub * 8 + i] = acc[h][i];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int h = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NSTATE; ++w) M = fmaxf(M, s_m[w][h]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < NSTATE; ++w) {
            const float f = s_m[w][h] == -INFINITY ? 0.f : expf(s_m[w][h] - M);
            L += s_l[w][h] * f;
            a += s_acc[w][h][d] * f;
        }
        if (n_splits == 1) {                      // the only range of its row: the result itself
            out[((size_t)t * nh + (size_t)g * G_all + h0 + h) * HD + d] = tq_from_float<TA>(a / L);
            continue;
        }
        float* dst = partial + (((size_t)t * nh + (size_t)g * G_all + h0 + h) * n_splits + split) * (HD + 2);
        dst[2 + d] = a;
        if (d == 0) { dst[0] = M; dst[1] = L; }
    }
    // The ring form never merges here: it serves launches of many short CTAs, which get a merge launch of their own,
    // and the mere presence of this call cost it 13 % (B200, 64 tokens x 16 heads x 4 ranges: 188 us against 167 us).
    if (STAGES > 0 || n_splits == 1 || arrived == nullptr) return;          // no tickets: attention_merge_kernel follows
    if constexpr (STAGES == 0) split_merge_by_last<TA, HD>(partial, n_splits, arrived + ((size_t)t * nkv + g) * chunks + chunk,
                                out + ((size_t)t * nh + (size_t)g * G_all + h0) * HD,
                                partial + ((size_t)t * nh + (size_t)g * G_all + h0) * n_splits * (HD + 2), G);
}

// The merge as a launch of its own, for launches of many short CTAs: there a fence and a ticket per CTA cost more than
// the second launch (measured on B200, 64 tokens x 16 heads x 4 ranges of 512 keys: 4.65 ms of split kernels per
// step with tickets against 3.95 + 0.10 ms with this kernel).  The same sums in the same order as the last CTA's.
template <typename TA>
__global__ void attention_merge_kernel(const float* __restrict__ partial, int n_splits, int hd, TA* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const size_t th = blockIdx.x;                        // token * nh + head
    const float* p = partial + th * n_splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p[(size_t)s * (hd + 2)]);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float L = 0.f, a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = p[(size_t)s * (hd + 2)];
            if (ms != -INFINITY) {
                const float f = expf(ms - M);
                L += p[(size_t)s * (hd + 2) + 1] * f;
                a += p[(size_t)s * (hd + 2) + 2 + d] * f;
            }
        }
        out[th * hd + d] = tq_from_float<TA>(a / L);
    }
}

// ---------------------------------------------------------------------------------------
// Split attention for grouped queries on tensor cores (bfloat16, head size 64 or 128, 3 to 16 query heads per KV
// head).  With several query heads per KV head the register form above is bound by its arithmetic, not by the
// stream of keys: every key costs 2 * head size multiply-adds PER QUERY HEAD on CUDA cores (measured on B200 at 7
// heads per KV head, 64 tokens x 4 KV heads x 2,048 keys: 165 us for 268 MB, 1.6 TB/s).  Here the query heads of a
// KV head are the 16 rows of one mma.sync tile (m16n8k16, bf16 in, fp32 out), so keys and values are read once per
// group and the arithmetic rides on the tensor pipe.  The op stays memory-bound and its M is 3..16 rows, which is why
// this is the warp-level mma and not tcgen05 (whose tiles start at 64 rows and want a CTA-wide TMEM pipeline).
//   grid (token, KV head, range) as above; a warp takes groups of 16 consecutive positions (never across a page),
//   brings each group's 16 key rows and 16 value rows into its own two-stage ring with 16-byte cp.async copies
//   (16-byte chunks XOR-swizzled by the row so that ldmatrix is conflict-free), computes S = Q K^T (scores in fp32,
//   scaled and masked there), keeps an online softmax per row in fp32, rounds P to bfloat16 as the A operand of
//   O += P V (as the prompt kernel does), and the warps' states are merged through shared memory into the same
//   partial-state format as the register form, so the merge (tickets or merge launch) is shared.
// ---------------------------------------------------------------------------------------
#define GQA_WARPS 4
#define GQA_STAGES 2
#define GQA_KEYS 16                              // positions per group

__device__ __forceinline__ void gqa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gqa_ldmatrix(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(smem_row)));
}
__device__ __forceinline__ void gqa_ldmatrix_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(smem_row)));
}
__device__ __forceinline__ uint32_t gqa_pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD> constexpr int gqa_smem_bytes() {
    // the ring: [warp][stage][K tile, V tile][16 rows][HD] bf16; reused by the merge: [warp][16 rows][HD + 2] floats
    constexpr int ring = GQA_WARPS * GQA_STAGES * 2 * GQA_KEYS * HD * 2;
    constexpr int merge = GQA_WARPS * 16 * (HD + 2) * 4;
    return ring > merge ? ring : merge;
}

template <int HD>
__global__ void __launch_bounds__(GQA_WARPS * 32)
attention_gqa_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                     const int* __restrict__ page_table, int table_stride, int page_size, int window, float scale,
                     float* __restrict__ partial, int n_splits, int* __restrict__ arrived,
                     __nv_bfloat16* __restrict__ out, int nh, int nkv, int n_seqs, int n_pages, int early_keys) {
    // early_keys: as in attention_split_kernel (a decode step: a warp's first group of keys, if it lies below the
    // token's own position, is asked for before the wait on the kernel ahead)
    if (!early_keys) {
        tq_grid_wait();                    // everything below may read what the previous kernel wrote
        tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    }
    constexpr int CPR = HD / 8;                          // 16-byte chunks per row
    constexpr int TILE = GQA_KEYS * HD;                  // elements of a K (or V) tile
    extern __shared__ __align__(128) unsigned char s_gqa[];
    const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int G = nh / nkv;                              // 3..16 rows of the tile are query heads, the rest zero
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;           // row of the fragments / column pair
    const int pos = positions[t];
    const int start = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = page_table + (size_t)TQ_CHECKED(seq_of_token[t], n_seqs, TQ_IDX_SEQUENCE) * table_stride;
    const int first = start / GQA_KEYS, last = pos / GQA_KEYS;          // inclusive groups of 16 positions
    const int groups = last - first + 1;
    const int per = (groups + n_splits - 1) / n_splits;
    const int gb = first + split * per, ge = min(last + 1, gb + per);

    float o[HD / 8][4];                                  // rows gid (0,1) and gid + 8 (2,3), head elements nd*8 + tig*2 + {0,1}
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) { o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;          // running maximum and this lane's share of the sum

    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(s_gqa) + (size_t)warp * GQA_STAGES * 2 * TILE;
    auto copy_group = [&](int grp, int stage) {
        const int p0 = grp * GQA_KEYS;
        const int page = TQ_CHECKED(table[TQ_CHECKED(p0 / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
        const __nv_bfloat16* kbase = cache + (((size_t)page * 2 + 0) * nkv + g) * page_size * HD + (size_t)(p0 % page_size) * HD;
        const __nv_bfloat16* vbase = kbase + (size_t)nkv * page_size * HD;
        __nv_bfloat16* kt = ring + (size_t)stage * 2 * TILE;
        __nv_bfloat16* vt = kt + TILE;
#pragma unroll
        for (int i = 0; i < GQA_KEYS * CPR / 32; ++i) {
            const int idx = lane + 32 * i, r = idx / CPR, c = idx % CPR;
            const int dst = (r * CPR + (c ^ (r & 7))) * 8;
            split_copy16(kt + dst, kbase + (size_t)r * HD + c * 8);
            split_copy16(vt + dst, vbase + (size_t)r * HD + c * 8);
        }
    };
    int next_grp = gb + warp, next_stage = 0, stage = 0;
    const bool keys_ahead = early_keys && next_grp * GQA_KEYS + GQA_KEYS - 1 < pos;    // the first group ends below the token's position
    if (early_keys && !keys_ahead) { tq_grid_wait(); tq_grid_launch_dependents(); }
    if (next_grp < ge) copy_group(next_grp, next_stage);
    split_commit();
    next_grp += GQA_WARPS;
    next_stage ^= 1;
    if (keys_ahead) { tq_grid_wait(); tq_grid_launch_dependents(); }
    // the queries as A fragments: rows gid and gid + 8 (heads), 16 head elements per k-step
    uint32_t qa[HD / 16][4];
    {
        // (keys and values come in by cp.async, volatile statements that keep their place behind the wait; the
        // queries are plain loads)
        const __nv_bfloat16* q0 = (early_keys ? tq_fresh(q) : q) + ((size_t)t * nh + (size_t)g * G + gid) * HD + tig * 2;
        const __nv_bfloat16* q1 = q0 + (size_t)8 * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qa[ks][0] = gid < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16) : 0u;
            qa[ks][1] = gid + 8 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16) : 0u;
            qa[ks][2] = gid < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8) : 0u;
            qa[ks][3] = gid + 8 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8) : 0u;
        }
    }
    for (int grp = gb + warp; grp < ge; grp += GQA_WARPS) {
        if (next_grp < ge) copy_group(next_grp, next_stage);          // the stage read one iteration ago
        split_commit();
        next_grp += GQA_WARPS;
        next_stage ^= 1;
        split_wait<1>();                                              // all but the newest group have landed: this one has
        __syncwarp();
        const __nv_bfloat16* kt = ring + (size_t)stage * 2 * TILE;
        const __nv_bfloat16* vt = kt + TILE;
        stage ^= 1;
        // ---- S = Q K^T: two tiles of 8 keys ----
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int mi = lane >> 3, key = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t b[4];
                const int chunk = ks * 2 + (mi & 1);
                gqa_ldmatrix(b, kt + (key * CPR + (chunk ^ (key & 7))) * 8);
                gqa_mma(s[0], qa[ks], b[0], b[1]);
                gqa_mma(s[1], qa[ks], b[2], b[3]);
            }
        }
        // ---- scale, mask, online softmax (rows gid and gid + 8; a row's 16 scores sit in the 4 lanes of a quad) ----
        const int p0 = grp * GQA_KEYS;
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int p = p0 + nt * 8 + tig * 2 + e;
                const bool seen = p >= start && p <= pos;
                s[nt][e] = seen ? s[nt][e] * scale : -INFINITY;
                s[nt][2 + e] = seen ? s[nt][2 + e] * scale : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // a group always holds a position its rows see (it lies between start and pos), so mx is finite here
        const float c0 = expf(m0 - mx0), c1 = expf(m1 - mx1);         // exp(-inf) = 0 the first time
        m0 = mx0; m1 = mx1;
        l0 *= c0; l1 *= c1;
        uint32_t pa[4];
        {
            const float e00 = expf(s[0][0] - mx0), e01 = expf(s[0][1] - mx0), e10 = expf(s[1][0] - mx0), e11 = expf(s[1][1] - mx0);
            const float f00 = expf(s[0][2] - mx1), f01 = expf(s[0][3] - mx1), f10 = expf(s[1][2] - mx1), f11 = expf(s[1][3] - mx1);
            l0 += (e00 + e01) + (e10 + e11);
            l1 += (f00 + f01) + (f10 + f11);
            pa[0] = gqa_pack(e00, e01);      // row gid,     keys tig*2 + {0,1}
            pa[1] = gqa_pack(f00, f01);      // row gid + 8, keys tig*2 + {0,1}
            pa[2] = gqa_pack(e10, e11);      // row gid,     keys 8 + tig*2 + {0,1}
            pa[3] = gqa_pack(f10, f11);      // row gid + 8, keys 8 + tig*2 + {0,1}
        }
        // ---- O = O * corr + P V ----
        {
            const int mi = lane >> 3, key = (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int nd = 0; nd < HD / 8; nd += 2) {
                uint32_t b[4];
                const int chunk = nd + (mi >> 1);
                gqa_ldmatrix_trans(b, vt + (key * CPR + (chunk ^ (key & 7))) * 8);
                o[nd][0] *= c0; o[nd][1] *= c0; o[nd][2] *= c1; o[nd][3] *= c1;
                o[nd + 1][0] *= c0; o[nd + 1][1] *= c0; o[nd + 1][2] *= c1; o[nd + 1][3] *= c1;
                gqa_mma(o[nd], pa, b[0], b[1]);
                gqa_mma(o[nd + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();                                                 // the stage may be overwritten two iterations on
    }
    split_wait<0>();
    // ---- the warps' states through shared memory (the ring is no longer needed) ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();
    float* st = reinterpret_cast<float*>(s_gqa) + (size_t)warp * 16 * (HD + 2);      // [row][m, l, HD values]
    if (tig == 0) {
        st[(size_t)gid * (HD + 2)] = m0; st[(size_t)gid * (HD + 2) + 1] = l0;
        st[(size_t)(gid + 8) * (HD + 2)] = m1; st[(size_t)(gid + 8) * (HD + 2) + 1] = l1;
    }
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
        float* r0 = st + (size_t)gid * (HD + 2) + 2 + nd * 8 + tig * 2;
        float* r1 = st + (size_t)(gid + 8) * (HD + 2) + 2 + nd * 8 + tig * 2;
        r0[0] = o[nd][0]; r0[1] = o[nd][1]; r1[0] = o[nd][2]; r1[1] = o[nd][3];
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(s_gqa);
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int h = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < GQA_WARPS; ++w) M = fmaxf(M, all[((size_t)w * 16 + h) * (HD + 2)]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < GQA_WARPS; ++w) {
            const float* sw = all + ((size_t)w * 16 + h) * (HD + 2);
            const float f = sw[0] == -INFINITY ? 0.f : expf(sw[0] - M);
            L += sw[1] * f;
            a += sw[2 + d] * f;
        }
        if (n_splits == 1) {
            out[((size_t)t * nh + (size_t)g * G + h) * HD + d] = __float2bfloat16_rn(a / L);
            continue;
        }
        float* dst = partial + (((size_t)t * nh + (size_t)g * G + h) * n_splits + split) * (HD + 2);
        dst[2 + d] = a;
        if (d == 0) { dst[0] = M; dst[1] = L; }
    }
    if (n_splits == 1 || arrived == nullptr) return;          // no tickets: attention_merge_kernel follows
    split_merge_by_last<__nv_bfloat16, HD>(partial, n_splits, arrived + (size_t)t * nkv + g,
                                           out + ((size_t)t * nh + (size_t)g * G) * HD,
                                           partial + ((size_t)t * nh + (size_t)g * G) * n_splits * (HD + 2), G);
}

// partial: T * nh * n_splits * (hd + 2) floats of scratch; arrived: T * nkv * ceil(G / 8) ints (G = nh / nkv) that are
// zero before the launch and zero again after it (both unused, and may be null, with one range).  early_keys: the
// caller vouches that the kernel ahead of this one in the stream wrote nothing this launch reads but the queries and
// the keys and values at the tokens' own positions (a decode step: one new token per sequence); older keys are then
// asked for before the wait on that kernel.
TQ_EXPORT int tq_attention_split(const void* q, const void* cache, int act_dtype, const int* positions,
                                 const int* seq_of_token, const int* page_table, int table_stride, int page_size,
                                 int window, float scale, float* partial, int n_splits, int* arrived, void* out, int T_,
                                 int nh, int nkv, int hd, int n_seqs, int n_pages, int early_keys, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd == 16 || hd == 32 || hd == 64 || hd == 128 || hd == 256,
               "attention_split: head size %d is not 16, 32, 64, 128 or 256", hd);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "attention_split: %d heads are not a multiple of %d key/value heads", nh, nkv);
    const int G = nh / nkv;
    // query heads per KV head a CTA keeps in registers: all of them up to 8; more are shared out in chunks of 8.
    // (With 7 heads the arithmetic, not the stream, bounds the kernel: 1,792 fp32 multiply-adds per key.  Measured
    // on B200 at 64 tokens x 4 KV heads x 2,048 keys: 165 us with 8 heads per CTA, 176 us with chunks of 4.)
    const int gc = G == 1 ? 1 : (G == 2 ? 2 : (G <= 4 ? 4 : 8));
    const int chunks = (G + gc - 1) / gc;
    TQ_REQUIRE((long long)T_ * chunks <= 0x7fffffffLL, "attention_split: %d tokens x %d head chunks exceed the grid", T_, chunks);
    TQ_REQUIRE(page_size % 16 == 0, "attention_split: page size %d must be a multiple of 16", page_size);
    TQ_REQUIRE(n_splits >= 1 && n_splits <= 65535 && nkv <= 65535, "attention_split: bad grid (%d splits, %d KV heads)", n_splits, nkv);
    TQ_REQUIRE(window >= 0, "attention_split: negative window %d", window);
    TQ_REQUIRE(n_splits == 1 || (partial != nullptr && arrived != nullptr),
               "attention_split: %d ranges need scratch for their partial states and their tickets", n_splits);
    // one launch with tickets while the CTAs fit about two waves (there the second launch is what costs), a merge
    // launch of its own for more and shorter CTAs
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
            || sm_count <= 0)
            TQ_FAIL(-1, "attention_split: cannot read the device's SM count");
    }
    const long long n_ctas = (long long)T_ * chunks * nkv * n_splits;
    dim3 grid(T_ * chunks, nkv, n_splits);
    // the ring form for launches of more than two waves of the register form (TQ_SPLIT_RING=1: wherever the
    // shape has one, =0: never)
    const char* ring_env = getenv("TQ_SPLIT_RING");
    const bool ring = ring_env && ring_env[0] ? ring_env[0] != '0' : n_ctas > 2LL * SPLIT_REGISTER_CTAS_PER_SM * sm_count;
    const bool own_merge = n_splits > 1 && (n_ctas > 2LL * SPLIT_REGISTER_CTAS_PER_SM * sm_count || ring);
    if (own_merge) arrived = nullptr;
    // grouped queries in bfloat16: the tensor-core form (TQ_NO_GQA_MMA=1: the register form everywhere)
    static const bool gqa_mma = [] { const char* e = getenv("TQ_NO_GQA_MMA"); return !(e && e[0] && e[0] != '0'); }();
    if (gqa_mma && act_dtype == TQ_BF16 && (hd == 64 || hd == 128) && G >= 3 && G <= 16) {
#define GQA_LAUNCH(HD_)                                                                                         \
        do {                                                                                                    \
            auto kern = attention_gqa_kernel<HD_>;                                                              \
            constexpr int smem = gqa_smem_bytes<HD_>();                                                         \
            static bool configured = false;                                                                     \
            if (!configured) {                                                                                  \
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);  \
                if (e != cudaSuccess) TQ_FAIL(-1, "attention_split: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e)); \
                configured = true;                                                                              \
            }                                                                                                   \
            tq_launch(dim3(T_, nkv, n_splits), GQA_WARPS * 32, smem, stream)(kern,                              \
                (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, positions, seq_of_token, page_table, table_stride, \
                page_size, window, scale, partial, n_splits, arrived, (__nv_bfloat16*)out, nh, nkv, n_seqs, n_pages, early_keys); \
        } while (0)
        if (hd == 64) GQA_LAUNCH(64); else GQA_LAUNCH(128);
#undef GQA_LAUNCH
        TQ_CHECK_LAUNCH("attention_gqa");
        if (own_merge) {
            tq_launch(T_ * nh, hd >= 128 ? 128 : 64, 0, stream)(attention_merge_kernel<__nv_bfloat16>, partial, n_splits, hd, (__nv_bfloat16*)out);
            TQ_CHECK_LAUNCH("attention_merge");
        }
        return 0;
    }
#define SPLIT_LAUNCH(TA, LPK, GC, STAGES)                                                                       \
    do {                                                                                                        \
        auto kern = attention_split_kernel<TA, LPK, GC, STAGES>;                                                \
        constexpr int ring = split_ring_bytes<TA, LPK, STAGES>();                                               \
        static bool configured = false;                                                                         \
        if (ring > 0 && !configured) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ring);      \
            if (e != cudaSuccess) TQ_FAIL(-1, "attention_split: %d bytes of shared memory refused: %s", ring, cudaGetErrorString(e)); \
            configured = true;                                                                                  \
        }                                                                                                       \
        tq_launch(grid, SPLIT_WARPS * 32, ring, stream)(kern,                                                   \
            (const TA*)q, (const TA*)cache, positions, seq_of_token, page_table, table_stride, page_size, window, \
            scale, partial, n_splits, arrived, (TA*)out, nh, nkv, n_seqs, n_pages, early_keys);                 \
    } while (0)
#define SPLIT_GC(TA, LPK)                                                                                       \
    do { if (G == 1) { if (ring && split_stages<TA, LPK>() > 0) SPLIT_LAUNCH(TA, LPK, 1, (split_stages<TA, LPK>()));   \
                       else SPLIT_LAUNCH(TA, LPK, 1, 0); }                                                      \
         else if (G == 2) SPLIT_LAUNCH(TA, LPK, 2, 0);                                                          \
         else if (G <= 4) SPLIT_LAUNCH(TA, LPK, 4, 0); else SPLIT_LAUNCH(TA, LPK, 8, 0); } while (0)
#define SPLIT_HD(TA)                                                                                            \
    do { if (hd == 16) SPLIT_GC(TA, 2); else if (hd == 32) SPLIT_GC(TA, 4); else if (hd == 64) SPLIT_GC(TA, 8);         \
         else if (hd == 128) SPLIT_GC(TA, 16); else SPLIT_GC(TA, 32); } while (0)
    if (act_dtype == TQ_BF16) SPLIT_HD(__nv_bfloat16);
    else if (act_dtype == TQ_F32) SPLIT_HD(float);
    else TQ_FAIL(-2, "attention_split: unknown element type %d", act_dtype);
    TQ_CHECK_LAUNCH("attention_split");
    if (own_merge) {
        TQ_DISPATCH(act_dtype, TA,
            (tq_launch(T_ * nh, hd >= 128 ? 128 : 64, 0, stream)(attention_merge_kernel<TA>, partial, n_splits, hd, (TA*)out)));
        TQ_CHECK_LAUNCH("attention_merge");
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// The same split attention with its scratch inside the library (see attention_no_alloc.h): for
// callers that cannot allocate device memory.  In host code `tq_static_partial` is only a stand-in
// for the symbol; its device address comes from cudaGetSymbolAddress, once per device.
// ---------------------------------------------------------------------------------------
#include "attention_no_alloc.h"

static __device__ __align__(256) float tq_static_partial[TQ_ATTENTION_STATIC_SCRATCH_FLOATS];
// tickets of the (token, KV head) rows: zero when the library is loaded, and every launch leaves them zero
static __device__ __align__(256) int tq_static_arrived[TQ_ATTENTION_STATIC_ROWS];

#define TQ_MAX_DEVICES 64
// device addresses of the two arrays, per device.  Two host threads making a device's first call at the same time
// both look the addresses up and store the same values: harmless.
static float* tq_static_partial_addr[TQ_MAX_DEVICES];
static int* tq_static_arrived_addr[TQ_MAX_DEVICES];

TQ_EXPORT int tq_attention_split_static(const void* q, const void* cache, int act_dtype, const int* positions,
                                        const int* seq_of_token, const int* page_table, int table_stride,
                                        int page_size, int window, float scale, int n_splits, void* out, int T_,
                                        int nh, int nkv, int hd, cudaStream_t stream) {
    // the caller's tables are taken as they are: a debug build's index checks get limits that nothing exceeds
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && nh > 0 && n_splits > 0 && hd > 0, "attention_split_static: bad sizes T=%d nh=%d splits=%d hd=%d",
               T_, nh, n_splits, hd);
    const unsigned long long need = (unsigned long long)T_ * nh * n_splits * (hd + 2);
    TQ_REQUIRE(need <= (unsigned long long)TQ_ATTENTION_STATIC_SCRATCH_FLOATS,
               "attention_split_static: %llu floats of scratch needed (T=%d, heads=%d, splits=%d, head size=%d) but the "
               "built-in array holds %d; use tq_attention_split with a buffer of your own",
               need, T_, nh, n_splits, hd, TQ_ATTENTION_STATIC_SCRATCH_FLOATS);
    TQ_REQUIRE(nkv > 0 && (long long)T_ * nh <= TQ_ATTENTION_STATIC_ROWS,
               "attention_split_static: %lld (token, head) rows exceed the %d the built-in ticket array holds; use "
               "tq_attention_split with buffers of your own", (long long)T_ * nh, TQ_ATTENTION_STATIC_ROWS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) TQ_FAIL(-1, "attention_split_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    TQ_REQUIRE(device >= 0 && device < TQ_MAX_DEVICES, "attention_split_static: device %d is beyond %d", device, TQ_MAX_DEVICES);
    if (tq_static_partial_addr[device] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, tq_static_partial);
        if (e != cudaSuccess || p == nullptr)
            TQ_FAIL(-1, "attention_split_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        int* a = nullptr;
        e = cudaGetSymbolAddress((void**)&a, tq_static_arrived);
        if (e != cudaSuccess || a == nullptr)
            TQ_FAIL(-1, "attention_split_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        tq_static_arrived_addr[device] = a;
        tq_static_partial_addr[device] = p;
    }
    return tq_attention_split(q, cache, act_dtype, positions, seq_of_token, page_table, table_stride, page_size, window,
                              scale, tq_static_partial_addr[device], n_splits, tq_static_arrived_addr[device], out, T_, nh,
                              nkv, hd, 0x7fffffff, 0x7fffffff, 0, stream);
}

// ---------------------------------------------------------------------------------------
// Tiled attention for runs of new tokens where the tensor-core prompt kernel does not apply (float32, or head
// sizes other than 64 and 128): a CTA takes 32 consecutive new tokens of one sequence and one query head, walks
// the keys they see in tiles of 64 through shared memory, and keeps an online softmax per row.  Keys and values
// are read once per 32 queries instead of once per query.  All arithmetic is IEEE fp32 on CUDA cores (fmaf,
// expf); nothing is rounded below fp32 on the way except what the cache's own element type stores.
//   warp w owns rows 8w..8w+7 of the query tile; for the scores a lane owns keys `lane` and `lane + 32` of the key tile, for the
//   weighted sum of values it owns head elements lane, lane+32, ...
// Row t of q belongs to the sequence i with cu_seqlens[i] <= t < cu_seqlens[i+1] and sits at position
// seq_start[i] + (t - cu_seqlens[i]); the step's keys and values are already in the cache.
// ---------------------------------------------------------------------------------------
#define TILED_BQ 32
#define TILED_BK 64                               // two keys per lane
#define TILED_WARPS 4
#define TILED_ROWS (TILED_BQ / TILED_WARPS)       // query rows per warp
#define TILED_MAX_EPL (TQ_MAX_HEAD_DIM / 32)      // head elements per lane, at most

__device__ __forceinline__ float4 tiled_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 tiled_load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// EPL: head elements per lane that the instantiation provides for (head size <= 32 * EPL)
template <typename TA, int EPL>
__global__ void __launch_bounds__(TILED_WARPS * 32)
attention_tiled_kernel(const TA* __restrict__ q, const TA* __restrict__ cache, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_start, const int* __restrict__ page_table, int table_stride,
                       int page_size, int window, float scale, TA* __restrict__ out, int n_seqs, int nh, int nkv,
                       int hd, int n_pages) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ __align__(16) float s_tiled[];
    const int ks = hd + 4;                                   // row stride of the key and query tiles (16-byte rows, no bank conflicts)
    float* s_q = s_tiled;                                    // [BQ][ks], scaled
    float* s_k = s_q + TILED_BQ * ks;                        // [BK][ks]
    float* s_v = s_k + TILED_BK * ks;                        // [BK][hd]
    float* s_p = s_v + TILED_BK * hd;                        // [WARPS][BK][ROWS]
    __shared__ int s_seq, s_row0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {                                  // which sequence's which 32 rows this CTA takes
        // later rows of a sequence see more keys: they are handed out first, so that the launch does not end
        // with its longest tiles
        int tile = blockIdx.x, seq = -1, row0 = 0;
        for (int i = 0; i < n_seqs; ++i) {
            const int n = cu_seqlens[i + 1] - cu_seqlens[i], tiles = (n + TILED_BQ - 1) / TILED_BQ;
            if (tile < tiles) { seq = i; row0 = (tiles - 1 - tile) * TILED_BQ; break; }
            tile -= tiles;
        }
        s_seq = seq; s_row0 = row0;
    }
    __syncthreads();
    const int seq = s_seq;
    if (seq < 0) return;                                     // the grid is an upper bound of the number of tiles
    const int h = blockIdx.y, g = h / (nh / nkv);
    const int t_first = cu_seqlens[seq] + s_row0;
    const int rows = min(TILED_BQ, cu_seqlens[seq + 1] - t_first);
    const int pos0 = seq_start[seq] + s_row0;                // position of the tile's first row
    const int* table = page_table + (size_t)seq * table_stride;
    for (int idx = threadIdx.x; idx < TILED_BQ * hd; idx += blockDim.x) {
        const int r = idx / hd, d = idx - r * hd;
        s_q[r * ks + d] = r < rows ? tq_to_float(q[((size_t)(t_first + r) * nh + h) * hd + d]) * scale : 0.f;
    }
    float m[TILED_ROWS], l[TILED_ROWS], acc[TILED_ROWS][EPL];
#pragma unroll
    for (int r = 0; r < TILED_ROWS; ++r) {
        m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int c = 0; c < EPL; ++c) acc[r][c] = 0.f;
    }
    // keys any row of the tile sees: from the first row's window start to the last row's own position
    const int k_lo = window > 0 ? max(0, pos0 + 1 - window) : 0, k_hi = pos0 + rows - 1;
    float* my_p = s_p + warp * TILED_BK * TILED_ROWS;
    const float* my_q = s_q + warp * TILED_ROWS * ks;
    for (int k0 = (k_lo / TILED_BK) * TILED_BK; k0 <= k_hi; k0 += TILED_BK) {
        __syncthreads();                                     // the previous tile has been used (and s_q is complete)
#pragma unroll 4
        for (int idx = threadIdx.x; idx < TILED_BK * (hd / 4); idx += blockDim.x) {
            const int j = idx / (hd / 4), d = (idx - j * (hd / 4)) * 4;
            const int p = k0 + j;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (p <= k_hi && p >= k_lo) {
                const int page = TQ_CHECKED(table[TQ_CHECKED(p / page_size, table_stride, TQ_IDX_TABLE_COLUMN)], n_pages, TQ_IDX_PAGE);
                const TA* kp = cache + ((((size_t)page * 2 + 0) * nkv + g) * page_size + p % page_size) * hd + d;
                kv = tiled_load4(kp);                        // hd is a multiple of 4: rows of 4 elements are aligned
                vv = tiled_load4(kp + (size_t)nkv * page_size * hd);
            }
            *reinterpret_cast<float4*>(s_k + j * ks + d) = kv;
            *reinterpret_cast<float4*>(s_v + j * hd + d) = vv;
        }
        __syncthreads();
        // scores of this warp's rows against keys `lane` and `lane + 32` of the tile
        float s0[TILED_ROWS], s1[TILED_ROWS];
#pragma unroll
        for (int r = 0; r < TILED_ROWS; ++r) { s0[r] = 0.f; s1[r] = 0.f; }
        const float* krow0 = s_k + lane * ks;
        const float* krow1 = krow0 + 32 * ks;
#pragma unroll 2
        for (int d = 0; d < hd; d += 4) {
            const float4 ka = *reinterpret_cast<const float4*>(krow0 + d);
            const float4 kb = *reinterpret_cast<const float4*>(krow1 + d);
#pragma unroll
            for (int r = 0; r < TILED_ROWS; ++r) {
                const float4 qq = *reinterpret_cast<const float4*>(my_q + r * ks + d);
                s0[r] = fmaf(qq.x, ka.x, s0[r]); s1[r] = fmaf(qq.x, kb.x, s1[r]);
                s0[r] = fmaf(qq.y, ka.y, s0[r]); s1[r] = fmaf(qq.y, kb.y, s1[r]);
                s0[r] = fmaf(qq.z, ka.z, s0[r]); s1[r] = fmaf(qq.z, kb.z, s1[r]);
                s0[r] = fmaf(qq.w, ka.w, s0[r]); s1[r] = fmaf(qq.w, kb.w, s1[r]);
            }
        }
        const int pa = k0 + lane, pb = pa + 32;
#pragma unroll
        for (int r = 0; r < TILED_ROWS; ++r) {
            const int row = warp * TILED_ROWS + r, pos = pos0 + row;
            const int start = window > 0 ? max(0, pos + 1 - window) : 0;
            const float sa = row < rows && pa >= start && pa <= pos ? s0[r] : -INFINITY;
            const float sb = row < rows && pb >= start && pb <= pos ? s1[r] : -INFINITY;
            const float mx = fmaxf(m[r], tq_warp_max(fmaxf(sa, sb)));
            float ea = 0.f, eb = 0.f, corr = 1.f;
            if (mx != -INFINITY) {                           // something of this row is visible by now
                corr = expf(m[r] - mx);                      // exp(-inf) = 0 the first time
                ea = expf(sa - mx);                          // exp(-inf) = 0 for what the row does not see
                eb = expf(sb - mx);
                l[r] = l[r] * corr + tq_warp_sum(ea + eb);
                m[r] = mx;
            }
#pragma unroll
            for (int c = 0; c < EPL; ++c) acc[r][c] *= corr;
            my_p[lane * TILED_ROWS + r] = ea;
            my_p[(lane + 32) * TILED_ROWS + r] = eb;
        }
        __syncwarp();
        // weighted sum of the tile's values: this lane's head elements, this warp's rows
#pragma unroll 2
        for (int j = 0; j < TILED_BK; ++j) {
            float pj[TILED_ROWS];
#pragma unroll
            for (int r = 0; r < TILED_ROWS; r += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(my_p + j * TILED_ROWS + r);
                pj[r] = t4.x; pj[r + 1] = t4.y; pj[r + 2] = t4.z; pj[r + 3] = t4.w;
            }
#pragma unroll
            for (int c = 0; c < EPL; ++c) {
                const int d = lane + 32 * c;
                if (d < hd) {
                    const float vv = s_v[j * hd + d];
#pragma unroll
                    for (int r = 0; r < TILED_ROWS; ++r) acc[r][c] = fmaf(pj[r], vv, acc[r][c]);
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < TILED_ROWS; ++r) {
        const int row = warp * TILED_ROWS + r;
        if (row >= rows) continue;
        TA* op = out + ((size_t)(t_first + row) * nh + h) * hd;
        const float inv = 1.0f / l[r];
#pragma unroll
        for (int c = 0; c < EPL; ++c) {
            const int d = lane + 32 * c;
            if (d < hd) op[d] = tq_from_float<TA>(acc[r][c] * inv);
        }
    }
}

// T_: rows of q; n_tiles_bound: an upper bound of the number of 32-row tiles (T_ / 32 + n_seqs serves).
TQ_EXPORT int tq_attention_tiled(const void* q, const void* cache, int act_dtype, const int* cu_seqlens,
                                 const int* seq_start, const int* page_table, int table_stride, int page_size,
                                 int window, float scale, void* out, int T_, int n_seqs, int nh, int nkv, int hd,
                                 int n_pages, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(hd % 4 == 0 && hd >= 4 && hd <= TQ_MAX_HEAD_DIM, "attention_tiled: head size %d must be a multiple of 4, at most %d", hd, TQ_MAX_HEAD_DIM);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "attention_tiled: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE(nh <= 65535 && n_seqs >= 1, "attention_tiled: bad grid (%d heads, %d sequences)", nh, n_seqs);
    TQ_REQUIRE(window >= 0, "attention_tiled: negative window %d", window);
    const size_t smem = ((size_t)(TILED_BQ + TILED_BK) * (hd + 4) + (size_t)TILED_BK * hd + TILED_WARPS * TILED_BK * TILED_ROWS) * sizeof(float);
    dim3 grid(T_ / TILED_BQ + n_seqs, nh);
#define TILED_LAUNCH(TA, EPL)                                                                                   \
    do {                                                                                                        \
        auto kern = attention_tiled_kernel<TA, EPL>;                                                            \
        static size_t configured = 0;                                                                           \
        if (smem > 48 * 1024 && smem > configured) {                                                            \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) TQ_FAIL(-1, "attention_tiled: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e)); \
            configured = smem;                                                                                  \
        }                                                                                                       \
        tq_launch(grid, TILED_WARPS * 32, smem, stream)(kern, (const TA*)q, (const TA*)cache, cu_seqlens, seq_start, \
            page_table, table_stride, page_size, window, scale, (TA*)out, n_seqs, nh, nkv, hd, n_pages);        \
    } while (0)
#define TILED_EPL(TA) do { if (hd <= 64) TILED_LAUNCH(TA, 2); else if (hd <= 128) TILED_LAUNCH(TA, 4); else TILED_LAUNCH(TA, TILED_MAX_EPL); } while (0)
    if (act_dtype == TQ_BF16) TILED_EPL(__nv_bfloat16);
    else if (act_dtype == TQ_F32) TILED_EPL(float);
    else TQ_FAIL(-2, "attention_tiled: unknown element type %d", act_dtype);
    TQ_CHECK_LAUNCH("attention_tiled");
    return 0;
}
