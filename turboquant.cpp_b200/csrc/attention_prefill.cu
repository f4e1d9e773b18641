// Causal attention for prompts on the 5th-generation tensor cores: S = Q K^T and O = P V as
// tcgen05.mma with the accumulators in tensor memory, Q/K/V tiles brought in by TMA straight from
// the query buffer and the paged key/value cache, online softmax in fp32 registers.
//
// Same mathematics as the exact kernel (csrc/attention.cu) and as the reference's per-token loop
// (src/engine/tq_transformer.c:1909-1936 scores with scale 1/sqrt(hd), :1960 softmax, :2183-2191
// weighted sum of V, head h reading KV head h/(nh/nkv) :1679, window start :1646-1654): scores,
// running maximum, sum and the output accumulator are fp32; only P is rounded to bf16 to feed the
// second product.
//
// A unit of work = 128 consecutive query tokens of one sequence x one query head; persistent CTAs (one per SM)
// each take several, heavy and light ones alternating, and walk a unit's keys in tiles of 128 (= two cache
// pages; the last tile may hold one).  While one unit's result is divided and written out, the next unit's
// Q is already loaded and its products run into the second O buffer:
//   warp 0        TMA: Q once, then K and V pages through two-stage rings
//   warp 1        owns tensor memory, issues  S = Q K^T  (M 128, N 128, K hd) one tile ahead into one
//                 of two S buffers, and  O += P V  (M 128, N hd, K 128; V is the MN-major operand, read
//                 as stored), accumulating in tensor memory over all key tiles
//   warps 2..9    two threads per query row (each warp reads its quarter of the tensor-memory lanes;
//                 the two threads of a row split the tile's 64 keys and the head's elements): read S,
//                 mask, online softmax, write P (bf16, 128-byte swizzled) to one of two buffers in
//                 shared memory.  O stays in tensor memory: it is rescaled there only when a row's
//                 maximum grows by more than 2^8 over the one its exponentials are taken against
//                 (until then P is simply larger, at most 256, and the row's sum carries the same
//                 factor), so a tile's softmax never waits for the products before it.
// Every wait on an mbarrier is bounded; a wait that runs out sets *status and the CTA
// leaves cleanly.
#include <cuda.h>
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

namespace {

constexpr int BM = 128;      // query rows per CTA
constexpr int THREADS = 320;   // TMA warp, MMA warp, eight softmax warps
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr uint64_t WAIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    uint64_t t0 = 0;
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_NS) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// K-major operand, rows of 128 bytes, 128-byte swizzle (see csrc/gemm_tc.cu)
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V as stored: one key per 128-byte row of 64 head elements): leading byte offset =
// distance between blocks of 64 head elements, stride byte offset = eight keys (1024 bytes)
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D fp32, A/B bf16, M 128, N n; b_mn: B is MN-major
__device__ __forceinline__ uint32_t idesc(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 2^x, one MUFU instruction; 2^-inf = 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

constexpr int PAGE = 64;     // tokens per cache page
constexpr int BN = 128;      // keys per tile = two cache pages (the last tile of a CTA may hold one)

template <int HD>
struct Cfg {
    static constexpr int HALVES = HD / 64;                 // 64-element (128-byte) column blocks of a head
    static constexpr int Q_BYTES = BM * HD * 2;
    static constexpr int PAGE_BYTES = PAGE * HD * 2;       // one page of K or of V for one KV head
    static constexpr int KV_BYTES = BN * HD * 2;           // a tile of K or of V
    static constexpr int P_BYTES = BM * BN * 2;
    static constexpr int STAGES = 2;                       // K and V tiles in flight
    static constexpr int TILE_BYTES = Q_BYTES + 2 * STAGES * KV_BYTES + 2 * P_BYTES;
    static constexpr int SUMS_BYTES = 2 * BM * 4;          // the two threads of a row exchange their sums here
    static constexpr int SMEM_BYTES = TILE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + SUMS_BYTES;
    static constexpr int TMEM_COLS = 512;                  // S twice (2 x 128 columns), O twice (2 x HD columns)
    static_assert(HD == 64 || HD == 128, "head size 64 or 128");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

// A unit of work: 128 consecutive query tokens of one sequence x one query head.
struct Item { int seq, h, t0, rows, p_first, pg_first, n_pages, n_tiles; bool valid; };

// Units are numbered with the query tile slowest and last tiles first (they see the most keys), and dealt to the
// CTAs in rounds that alternate direction (0..G-1, then G-1..0, ...), so every CTA gets a heavy and a light one.
__device__ __forceinline__ int unit_of_round(int round, int cta, int n_ctas) {
    return round * n_ctas + ((round & 1) ? n_ctas - 1 - cta : cta);
}
__device__ __forceinline__ Item item_of(int unit, int n_qt, int n_seqs, int nh, const int* cu_seqlens, const int* seq_start,
                                        int window) {
    Item it;
    const int per_qt = n_seqs * nh;
    const int x = unit / per_qt, rem = unit - x * per_qt;
    it.seq = rem / nh;
    it.h = rem - it.seq * nh;
    const int qt = n_qt - 1 - x;
    const int t_begin = cu_seqlens[it.seq], t_end = cu_seqlens[it.seq + 1];
    it.t0 = t_begin + qt * BM;
    it.valid = it.t0 < t_end;
    it.rows = min(BM, t_end - it.t0);
    it.p_first = seq_start[it.seq] + qt * BM;              // position of row 0
    const int p_last = it.p_first + it.rows - 1;
    const int lo = window > 0 ? max(0, it.p_first + 1 - window) : 0;
    it.pg_first = lo / PAGE;                               // cache pages this unit reads
    it.n_pages = it.valid ? p_last / PAGE - it.pg_first + 1 : 0;
    it.n_tiles = (it.n_pages + 1) / 2;
    return it;
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ page_table, int table_stride, int window, float scale_log2e,
                         __nv_bfloat16* __restrict__ out, int nh, int nkv, int n_qt, int n_seqs,
                         int* __restrict__ status) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    using C = Cfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem_base;

    const int n_units = n_qt * n_seqs * nh;
    const int cta = blockIdx.x, n_ctas = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kv_group = nh / nkv;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = base;
    auto k_smem = [&](int s) { return base + C::Q_BYTES + s * C::KV_BYTES; };
    auto v_smem = [&](int s) { return base + C::Q_BYTES + (C::STAGES + s) * C::KV_BYTES; };
    auto p_smem = [&](int b) { return base + C::Q_BYTES + 2 * C::STAGES * C::KV_BYTES + b * C::P_BYTES; };
    const uint32_t bars = base + C::TILE_BYTES;
    constexpr int NS = C::STAGES;
    const uint32_t q_full = bars, q_free = bars + 8u;                     // Q of a unit is in / is no longer read
    auto k_full = [&](int s) { return bars + 8u * (2 + s); };
    auto k_empty = [&](int s) { return bars + 8u * (2 + NS + s); };
    auto v_full = [&](int s) { return bars + 8u * (2 + 2 * NS + s); };
    auto v_empty = [&](int s) { return bars + 8u * (2 + 3 * NS + s); };
    auto s_ready = [&](int b) { return bars + 8u * (2 + 4 * NS + b); };
    auto p_ready = [&](int b) { return bars + 8u * (4 + 4 * NS + b); };   // P of a tile is in its buffer (and S has been read)
    auto pv_done = [&](int b) { return bars + 8u * (6 + 4 * NS + b); };   // the products that read P buffer b are done
    const uint32_t sums_ready = bars + 8u * (8 + 4 * NS);                 // every softmax warp has written its rows' sums
    const uint32_t sums_read = bars + 8u * (9 + 4 * NS);                  // ... and has read its partners'
    static_assert((10 + 4 * NS) * 8 <= 256, "barriers");
    float* s_sums = reinterpret_cast<float*>(smem_raw + (bars + 256u - smem_u32(smem_raw)));

    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(q_full, 1);
        mbar_init(q_free, 1);
        mbar_init(sums_ready, 8);
        mbar_init(sums_read, 8);
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(s_ready(b), 1); mbar_init(p_ready(b), 8); mbar_init(pv_done(b), 1); }   // 8: one arrival per softmax warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&s_tmem_base)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // only now: a dependent kernel that took tensor memory first could starve a CTA of this grid that
    // had not allocated yet, and then wait forever for this grid to finish
    tq_grid_launch_dependents();
    auto tmem_s = [&](int b) { return s_tmem_base + (uint32_t)(b * BN); };              // S, twice: BN columns each
    auto tmem_o = [&](int b) { return s_tmem_base + (uint32_t)(2 * BN + b * HD); };     // O, twice: HD columns each

    // Every role walks the same units in the same order and counts tiles across units: tile number `ti` picks the
    // K/V stage (ti % STAGES), the S and P buffers (ti & 1) and the barriers' phases; unit number `it` picks the O
    // buffer (it & 1), so one unit's result is written out while the next unit's products accumulate.
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int ti = 0, it = 0;
            bool ok = true;
            for (int round = 0; ok; ++round) {
                const int unit = unit_of_round(round, cta, n_ctas);
                if (unit >= n_units) break;
                const Item u = item_of(unit, n_qt, n_seqs, nh, cu_seqlens, seq_start, window);
                if (!u.valid) continue;
                const int g = u.h / kv_group;
                const int* table = page_table + (size_t)u.seq * table_stride;
                // the products that read the previous unit's Q must be done
                if (it > 0 && !mbar_wait(q_free, (uint32_t)(it - 1) & 1u, &s_abort)) break;
                mbar_expect_tx(q_full, (uint32_t)C::Q_BYTES);
#pragma unroll
                for (int c = 0; c < C::HALVES; ++c) tma_load_2d(q_smem + c * (BM * 128), &map_q, u.h * HD + c * 64, u.t0, q_full);
                ++it;
                for (int i = 0; i < u.n_tiles; ++i, ++ti) {
                    const int s = ti % C::STAGES;
                    const uint32_t ph = (uint32_t)(ti / C::STAGES) & 1u;
                    const int np = min(2, u.n_pages - 2 * i);
                    const int page0 = table[u.pg_first + 2 * i], page1 = np > 1 ? table[u.pg_first + 2 * i + 1] : 0;
                    // a tile in shared memory: [column block of 64 elements][128 keys][128 bytes]; a page is 64 keys of it
                    if (!mbar_wait(k_empty(s), ph ^ 1u, &s_abort)) { ok = false; break; }
                    mbar_expect_tx(k_full(s), (uint32_t)(np * C::PAGE_BYTES));
                    for (int pg = 0; pg < np; ++pg) {
                        const int krow = (((pg ? page1 : page0) * 2 + 0) * nkv + g) * PAGE;
#pragma unroll
                        for (int c = 0; c < C::HALVES; ++c)
                            tma_load_2d(k_smem(s) + c * (BN * 128) + pg * (PAGE * 128), &map_kv, c * 64, krow, k_full(s));
                    }
                    if (!mbar_wait(v_empty(s), ph ^ 1u, &s_abort)) { ok = false; break; }
                    mbar_expect_tx(v_full(s), (uint32_t)(np * C::PAGE_BYTES));
                    for (int pg = 0; pg < np; ++pg) {
                        const int vrow = (((pg ? page1 : page0) * 2 + 1) * nkv + g) * PAGE;
#pragma unroll
                        for (int c = 0; c < C::HALVES; ++c)
                            tma_load_2d(v_smem(s) + c * (BN * 128) + pg * (PAGE * 128), &map_kv, c * 64, vrow, v_full(s));
                    }
                }
            }
            if (s_abort) {      // let the copies this thread started land before the CTA goes away (bounded)
                if (it > 0) for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(q_full, (uint32_t)(it - 1) & 1u); ++i) {}
                for (int i = ti > C::STAGES ? ti - C::STAGES : 0; i < ti; ++i) {
                    const uint32_t ph = (uint32_t)(i / C::STAGES) & 1u;
                    for (uint32_t j = 0; j < WAIT_LIMIT && !mbar_try_wait(k_full(i % C::STAGES), ph); ++j) {}
                    for (uint32_t j = 0; j < WAIT_LIMIT && !mbar_try_wait(v_full(i % C::STAGES), ph); ++j) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // A product of M = 128 costs some 130-145 cycles whatever its N up to 128: tiles of 128 keys make the
        // most of each one (8 products for S, 8 for O per 128 keys).  S = Q K^T of a tile is issued one tile ahead
        // of the P V product, across units too: two cursors walk the same sequence of tiles.
        if (lane == 0) {
            const uint32_t id_o = idesc(HD, 1);
            struct Cursor { int round, it, ti, i; Item u; bool live; };
            auto enter = [&](Cursor& c) {           // the next valid unit from c.round on
                c.live = false;
                for (;; ++c.round) {
                    const int unit = unit_of_round(c.round, cta, n_ctas);
                    if (unit >= n_units) return;
                    c.u = item_of(unit, n_qt, n_seqs, nh, cu_seqlens, seq_start, window);
                    if (c.u.valid) break;
                }
                c.i = 0;
                c.live = true;
            };
            auto advance = [&](Cursor& c) {
                ++c.ti;
                if (++c.i == c.u.n_tiles) { ++c.round; ++c.it; enter(c); }
            };
            Cursor qk{0, 0, 0, 0, Item{}, false}, pv{0, 0, 0, 0, Item{}, false};
            enter(qk);
            enter(pv);
            bool ok = true;
            auto issue_qk = [&]() -> bool {
                const int s = qk.ti % C::STAGES, b = qk.ti & 1;
                const int np = min(2, qk.u.n_pages - 2 * qk.i);
                if (qk.i == 0 && !mbar_wait(q_full, (uint32_t)qk.it & 1u, &s_abort)) return false;
                if (!mbar_wait(k_full(s), (uint32_t)(qk.ti / C::STAGES) & 1u, &s_abort)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t id_s = idesc(PAGE * np, 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k / 4) * (BM * 128) + (k % 4) * 32, koff = (k / 4) * (BN * 128) + (k % 4) * 32;
                    umma(tmem_s(b), desc_k_major(q_smem + off), desc_k_major(k_smem(s) + koff), id_s, k > 0 ? 1u : 0u);
                }
                umma_commit(s_ready(b));
                umma_commit(k_empty(s));
                if (qk.i == qk.u.n_tiles - 1) umma_commit(q_free);       // the unit's last read of Q
                advance(qk);
                return true;
            };
            if (qk.live) ok = issue_qk();
            while (pv.live && ok) {
                // the other S buffer is free: its tile's P was complete before the P V product before this one was issued
                if (qk.live) ok = issue_qk();
                if (!ok) break;
                const int s = pv.ti % C::STAGES, b = pv.ti & 1;
                ok = mbar_wait(p_ready(b), (uint32_t)(pv.ti >> 1) & 1u, &s_abort) &&
                     mbar_wait(v_full(s), (uint32_t)(pv.ti / C::STAGES) & 1u, &s_abort);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int steps = (PAGE / 16) * min(2, pv.u.n_pages - 2 * pv.i);   // 16 keys per product; a missing second page is not read
                const uint32_t acc = tmem_o(pv.it & 1);
                for (int k = 0; k < steps; ++k)                  // O += P V (a unit's first tile starts the sum)
                    umma(acc, desc_k_major(p_smem(b) + (k / 4) * (BM * 128) + (k % 4) * 32),
                         desc_mn_major(v_smem(s) + k * 2048, BN * 128), id_o, (pv.i > 0 || k > 0) ? 1u : 0u);
                umma_commit(pv_done(b));
                umma_commit(v_empty(s));
                advance(pv);
            }
        }
    } else {
        // ------------------------------ softmax: two threads per query row ------------------------------
        constexpr int HK = PAGE / 2, HDH = HD / 2;    // keys of a page and head elements of one thread
        constexpr float RESCALE_LOG2 = 8.0f;          // O is rescaled when a row's maximum has grown by more than 2^8
        const int quarter = warp & 3, part = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        int ti = 0, it = 0;
        bool ok = true;
        for (int round = 0; ok; ++round) {
            const int unit = unit_of_round(round, cta, n_ctas);
            if (unit >= n_units) break;
            const Item u = item_of(unit, n_qt, n_seqs, nh, cu_seqlens, seq_start, window);
            if (!u.valid) continue;
            const int qpos = u.p_first + r;
            const int start = window > 0 ? max(0, qpos + 1 - window) : 0;
            const uint32_t acc = tmem_o(it & 1);
            // m: the maximum the row's exponentials are taken against (both threads of a row hold the same);
            // l: the sum of this thread's keys' exponentials
            float m = -INFINITY, l = 0.f;
            for (int i = 0; i < u.n_tiles && ok; ++i, ++ti) {
                const int b = ti & 1;
                const int np = min(2, u.n_pages - 2 * i);
                const int k0 = (u.pg_first + 2 * i) * PAGE;
                ok = __all_sync(0xffffffffu, mbar_wait(s_ready(b), (uint32_t)(ti >> 1) & 1u, &s_abort));   // warp-uniform
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // this thread's 32 keys of each page of the tile, and (for the maximum only) the other thread's
                uint32_t sv[2][32];
                float mx = m;
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (hf < np) {                                 // uniform across the CTA
                        uint32_t other[32];
                        tmem_ld32(tmem_s(b) + lane_addr + hf * PAGE + part * HK, sv[hf]);
                        tmem_ld32(tmem_s(b) + lane_addr + hf * PAGE + (1 - part) * HK, other);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        const int kh = k0 + hf * PAGE;
                        const bool visible = (kh + PAGE - 1 <= u.p_first) && (window == 0 || kh >= u.p_first + BM - window);
                        if (visible) {                             // every key of the page is seen by every row: no masking
#pragma unroll
                            for (int c = 0; c < HK; ++c)
                                mx = fmaxf(mx, fmaxf(__uint_as_float(sv[hf][c]), __uint_as_float(other[c])));
                        } else {
#pragma unroll
                            for (int c = 0; c < HK; ++c) {
                                const int kp = kh + part * HK + c, kq = kh + (1 - part) * HK + c;
                                float a = __uint_as_float(sv[hf][c]), bq = __uint_as_float(other[c]);
                                if (kp > qpos || kp < start) a = -INFINITY;
                                if (kq > qpos || kq < start) bq = -INFINITY;
                                sv[hf][c] = __float_as_uint(a);
                                mx = fmaxf(mx, fmaxf(a, bq));
                            }
                        }
                    }
                }
                // keep m unless the maximum grew by more than 2^8 (or nothing had been seen yet)
                float corr = 1.0f;
                if (m == -INFINITY) {
                    m = mx;                                // l and O are still zero: nothing to rescale
                } else if ((mx - m) * scale_log2e > RESCALE_LOG2) {
                    corr = ex2((m - mx) * scale_log2e);
                    l *= corr;
                    m = mx;
                }
                // the P buffer must be free (the products of two tiles ago are done), and O can only be rescaled
                // between the previous tile's products and this tile's
                if (ti >= 2) ok = __all_sync(0xffffffffu, mbar_wait(pv_done(b), (uint32_t)((ti >> 1) - 1) & 1u, &s_abort));
                if (!ok) break;
                if (__any_sync(0xffffffffu, corr != 1.0f)) {           // only with i > 0: the previous tile is this unit's
                    ok = __all_sync(0xffffffffu, mbar_wait(pv_done(b ^ 1), (uint32_t)((ti - 1) >> 1) & 1u, &s_abort));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int c0 = 0; c0 < HDH; c0 += 32) {
                        uint32_t ov[32];
                        tmem_ld32(acc + lane_addr + part * HDH + c0, ov);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * corr);
                        tmem_st32(acc + lane_addr + part * HDH + c0, ov);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                const float mref = m == -INFINITY ? 0.f : m * scale_log2e;   // nothing visible yet: exponents of -inf
                float lsum = 0.f;
                // P in bf16: [page of the tile][128 rows][128 bytes = 64 keys], 16-byte chunks of 8 keys written with
                // the 128-byte swizzle of a K-major operand
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (hf < np) {
                        const uint32_t prow = p_smem(b) + (uint32_t)hf * (BM * 128) + (uint32_t)(r / 8) * 1024u + (uint32_t)(r % 8) * 128u;
#pragma unroll
                        for (int ch = 0; ch < HK / 8; ++ch) {
                            uint32_t packed[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int c = ch * 8 + 2 * e;
                                const float a = ex2(fmaf(__uint_as_float(sv[hf][c]), scale_log2e, -mref));
                                const float bq = ex2(fmaf(__uint_as_float(sv[hf][c + 1]), scale_log2e, -mref));
                                lsum += a + bq;
                                const __nv_bfloat162 pk = __floats2bfloat162_rn(a, bq);
                                packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
                            }
                            const uint32_t dst = prow + (uint32_t)(((part * (HK / 8) + ch) ^ (r % 8)) * 16);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]),
                                         "r"(packed[2]), "r"(packed[3]) : "memory");
                        }
                    }
                }
                l += lsum;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready(b));
            }
            // the unit's products done: O / (the row's sum = the sum of its two threads' sums, same maximum m in both)
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_done((ti - 1) & 1), (uint32_t)((ti - 1) >> 1) & 1u, &s_abort));
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // (a warp may be here while another still reads the previous unit's sums: wait for those reads first)
            if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait(sums_read, (uint32_t)(it - 1) & 1u, &s_abort));
            s_sums[part * BM + r] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(sums_ready);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(sums_ready, (uint32_t)it & 1u, &s_abort));
            const float lrow = s_sums[r] + s_sums[BM + r];
            __syncwarp();
            if (lane == 0) mbar_arrive(sums_read);
            if (ok) {
                const float inv = 1.0f / lrow;
                __nv_bfloat16* dst = out + ((size_t)(u.t0 + r) * nh + u.h) * HD + part * HDH;
#pragma unroll
                for (int c0 = 0; c0 < HDH; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(acc + lane_addr + part * HDH + c0, ov);      // every lane takes part: the load is warp-wide
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (r < u.rows) {
#pragma unroll
                        for (int d = 0; d < 32; d += 8) {
                            uint32_t packed[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(ov[d + 2 * e]) * inv,
                                                                                __uint_as_float(ov[d + 2 * e + 1]) * inv);
                                packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
                            }
                            *reinterpret_cast<uint4*>(dst + c0 + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");   // the reads of O are ordered before the next arrivals
            }
            ++it;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(s_tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && s_abort) atomicExch(status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// bf16 matrix [rows][cols] row-major; box [box_rows][64 columns], 128-byte swizzle
int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) TQ_FAIL(-3, "attention_prefill: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TQ_FAIL(-3, "attention_prefill: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const int* cu, const int* starts, const int* table,
           int table_stride, int window, float scale, void* out, int n_seqs, int max_q_len, int nh, int nkv, int* status,
           cudaStream_t stream) {
    using C = Cfg<HD>;
    auto kern = attention_prefill_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) TQ_FAIL(-1, "attention_prefill: cannot reserve %d bytes of shared memory: %s", C::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    // persistent CTAs, one per SM at most: each walks its units (query tile x sequence x head)
    const int n_qt = (max_q_len + BM - 1) / BM;
    const long long units = (long long)n_qt * n_seqs * nh;
    const int grid = (int)(units < n_sm ? units : n_sm);
    tq_launch(grid, THREADS, C::SMEM_BYTES, stream)(kern, mq, mkv, cu, starts, table, table_stride, window,
                                                   scale * 1.4426950408889634f, (__nv_bfloat16*)out, nh, nkv, n_qt, n_seqs, status);
    TQ_CHECK_LAUNCH("attention_prefill");
    return 0;
}

}  // namespace

// q [T, nh, hd] bf16; cache [n_pages, 2, nkv, 64, hd] bf16 (keys and values of this step already written);
// out [T, nh*hd] bf16.  cu_seqlens [n_seqs+1]: rows of each sequence in q; seq_start [n_seqs]: position of
// each sequence's first row.  status: one int in device memory, set to 1 if a bounded wait ran out.
TQ_EXPORT int tq_attention_prefill(const void* q, const void* cache, const int* cu_seqlens, const int* seq_start,
                                   const int* page_table, int table_stride, int page_size, int n_pages, int window,
                                   float scale, void* out, int T_, int n_seqs, int max_q_len, int nh, int nkv, int hd,
                                   int* status, cudaStream_t stream) {
    if (T_ == 0 || n_seqs == 0) return 0;
    TQ_REQUIRE(hd == 64 || hd == 128, "attention_prefill: head size %d is not 64 or 128", hd);
    TQ_REQUIRE(page_size == PAGE, "attention_prefill: page size %d must be %d", page_size, PAGE);
    TQ_REQUIRE(nkv >= 1 && nh % nkv == 0, "attention_prefill: %d heads are not a multiple of %d key/value heads", nh, nkv);
    TQ_REQUIRE((long long)((max_q_len + BM - 1) / BM) * n_seqs * nh < (1ll << 30), "attention_prefill: too many units of work");
    TQ_REQUIRE(window >= 0 && max_q_len >= 1, "attention_prefill: bad window %d or longest run %d", window, max_q_len);
    TQ_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)cache % 16) == 0 && ((uintptr_t)out % 16) == 0,
               "attention_prefill: q, cache and out must be 16-byte aligned");
    TQ_REQUIRE(status != nullptr, "attention_prefill: a status word is required");
    CUtensorMap mq, mkv;
    int rc = make_map(&mq, q, (uint64_t)T_, (uint64_t)nh * hd, BM);
    if (rc) return rc;
    rc = make_map(&mkv, cache, (uint64_t)n_pages * 2 * nkv * PAGE, (uint64_t)hd, PAGE);
    if (rc) return rc;
    if (hd == 64)
        return launch<64>(mq, mkv, cu_seqlens, seq_start, page_table, table_stride, window, scale, out, n_seqs, max_q_len,
                          nh, nkv, status, stream);
    return launch<128>(mq, mkv, cu_seqlens, seq_start, page_table, table_stride, window, scale, out, n_seqs, max_q_len,
                       nh, nkv, status, stream);
}
