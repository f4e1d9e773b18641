// Grouped bf16 GEMM on the 5th-generation tensor cores (tcgen05) with TMA-fed shared memory and
// the accumulator in tensor memory: the expert products of the mixture-of-experts feed-forward
// (routed experts and the shared expert), for prompts and for decoding.
//
//   out[row, n] = sum_k X[row, k] * W[g(row), n, k]          (plain)
//   out[row, n] = silu(X.Wg[n]) * (X.Wu[n])                   (SwiGLU: W holds gate rows [0, N) and
//                                                              up rows [N, 2N) of each group)
// as the reference's expert loop computes them on the CPU (src/engine/tq_moe.c:975-999: g = Wg x,
// u = Wu x, h = silu(g)*u, o = Wd h); the SiLU's exponential and division are the exact ones for an fp32
// result and the fast ones (a few units in the last place of fp32) for a bfloat16 result.
//
// The weights are packed once at load time into [128 rows x 64 elements] blocks of 16 KiB, so a
// stage of the pipeline is one contiguous read and a CTA's stream walks memory sequentially instead
// of touching 128 rows 4 KiB apart (which thrashes DRAM row buffers when hundreds of CTAs stream).
// With SwiGLU a block holds 64 gate rows and the 64 up rows of the same output columns, interleaved
// in runs of 16 (rows 32q..32q+15: gate of columns 64j+16q.., rows 32q+16..32q+31: up of the same),
// so one MMA yields both halves of 64 outputs and an epilogue warp pairs them with one shuffle.
//
// Orientation: the WEIGHT rows are the M side of the MMA (128 rows per tile), the token rows are
// the N side: a tile has up to BN (16..256) token rows and the MMA's N is the tile's own row count
// rounded up to 16, so an expert with 136 rows costs one product of N = 144, not two of 128.  One
// kernel therefore serves a 2,048-token prompt and a decode step of a few tokens per expert without
// padding the tensor core's M dimension with empty rows: at decode the kernel is a weight stream
// (each CTA pulls a [128 x K] slab through a multi-stage TMA pipeline) and the tokens ride along as
// a narrow N.
//
// Persistent CTAs (one or two per SM) each walk a strided list of (weight-row tile, token tile)
// pairs.  Warp 0 issues the TMA loads of the weight blocks as one uninterrupted stream of k-blocks
// across tiles and warp 2 those of the token blocks (two rings of different depth), warp 1 owns
// the tensor memory and issues tcgen05.mma into one of two accumulators, warps 3.. read the other
// accumulator back (tcgen05.ld), apply the epilogue and store while the next tile is multiplied.
// Token tiles of 128 or 256 rows run on pairs of CTAs (cta_group::2): each CTA holds 128 weight rows
// and half of the token rows, the first CTA issues the products for both.
// All waits on mbarriers are bounded: a wait that runs out sets a flag, every
// role leaves its loop, copies in flight are waited for (bounded again), tensor memory is freed and
// the kernel returns with *status != 0; nothing spins forever.
#include <cuda.h>
#include <type_traits>
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

namespace {

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int BK = 64;           // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;       // K of one tcgen05.mma for 16-bit inputs
constexpr uint32_t WAIT_LIMIT = 1u << 20;     // polls of an mbarrier before a wait gives up
constexpr uint64_t WAIT_NS = 2000000000ull;   // ... or two seconds, whichever comes first

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
// Bounded wait.  Returns false when it gave up (and raises the CTA's abort flag) or when another
// role already gave up.
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

// L2 policies: weights of a prompt's or a step's experts are read once (evict first), token rows are read by
// every weight-row tile of their expert (evict last), so the weight stream does not push them out of the L2.
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
// one [128 rows x 64 elements] block of the packed weights: (k-block, tile) select the block
__device__ __forceinline__ void tma_load_block(uint32_t dst, const CUtensorMap* map, int kb, int tile, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(0), "r"(0), "r"(kb), "r"(tile), "l"(policy) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// start address >> 4, leading byte offset 1 (unused for swizzled K-major), stride byte offset
// 1024 >> 4 (eight rows), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// ---- CTA pairs (cta_group::2) ----------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// loads of a CTA pair: the data lands in this CTA, the bytes are counted on the barrier of the pair's first CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"((uint64_t)map), "r"(cluster_bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_load_block_pair(uint32_t dst, const CUtensorMap* map, int kb, int tile, uint32_t cluster_bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"((uint64_t)map), "r"(cluster_bar), "r"(0), "r"(0), "r"(kb), "r"(tile), "l"(policy) : "memory");
}
// one product of the pair: M = 256 (128 weight rows from each CTA), the token rows half from each CTA
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this address in both CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// silu(gate) * up.  A bfloat16 result keeps 8 bits, so the fast exponential and division (a few units in
// the last place of fp32) do; an fp32 result gets the exact ones.
template <typename TO> __device__ __forceinline__ float silu_mul(float gate, float up) {
    return gate / (1.0f + expf(-gate)) * up;
}
template <> __device__ __forceinline__ float silu_mul<__nv_bfloat16>(float gate, float up) {
    return __fdividef(gate, 1.0f + __expf(-gate)) * up;
}

template <int BN, bool PAIR>
struct Tile {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;       // token rows this CTA holds of a tile
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int BOX_ROWS = B_ROWS < 64 ? B_ROWS : 64;   // token rows of one TMA box; the tail comes in boxes of 16
    static constexpr int BOX_BYTES = BOX_ROWS * BK * 2;
    static constexpr int TAIL_ROWS = 16, TAIL_BYTES = TAIL_ROWS * BK * 2;

    // narrow token tiles (decoding) leave room for two CTAs per SM: one CTA's start-up and epilogue
    // overlap the other's weight stream; wide tiles take the whole SM
    static constexpr int CTAS_PER_SM = BN <= 32 ? 2 : 1;
    static constexpr int BUDGET = (CTAS_PER_SM == 2 ? 104 : 208) * 1024;
    // Two rings: weight blocks (16 KiB each) and token blocks.  Narrow token tiles: equally deep.  Wide ones:
    // the token blocks come from the L2 and a few slots cover its latency, while the weights of a prompt's
    // routed experts are read once from DRAM, whose latency under load (microseconds) needs as many
    // blocks in flight as fit; their loads run ahead of the token blocks' by the difference in depth.
    static constexpr int B_SLOTS = BN <= 64 ? ((BUDGET / (A_BYTES + B_BYTES)) > 8 ? 8 : BUDGET / (A_BYTES + B_BYTES))
                                            : (B_BYTES > 16 * 1024 ? 3 : 6);
    static constexpr int A_SLOTS = BN <= 64 ? B_SLOTS
                                            : ((BUDGET - B_SLOTS * B_BYTES) / A_BYTES > 12 ? 12 : (BUDGET - B_SLOTS * B_BYTES) / A_BYTES);
    // epilogue warps: one per quarter of the accumulator's lanes, two for wide tiles (each takes every other
    // group of 16 token rows), so that reading a tile back never takes longer than multiplying the next
    static constexpr int EPI_WARPS = BN >= 64 ? 8 : 4;
    static constexpr int THREADS = 96 + 32 * EPI_WARPS;        // two producers, the MMA issuer, the epilogue
    static constexpr int ACC_COLS = BN;
    // two accumulators in tensor memory: a tile's epilogue overlaps the next tile's products
    static constexpr int TMEM_COLS = 2 * ACC_COLS <= 32 ? 32 : (2 * ACC_COLS <= 64 ? 64 : (2 * ACC_COLS <= 128 ? 128 : (2 * ACC_COLS <= 256 ? 256 : 512)));
    static constexpr int SMEM_BYTES = A_SLOTS * A_BYTES + B_SLOTS * B_BYTES + 1024 /* alignment slack */ + 512 /* barriers */;
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "token tile must be 16..256 in steps of 16");
    static_assert(!PAIR || BN >= 128, "pairs are for wide token tiles");
    static_assert(B_SLOTS >= 2 && A_SLOTS >= B_SLOTS, "pipeline needs at least two stages");
    static_assert((2 * A_SLOTS + 4) * 8 <= 512, "barriers");
    static_assert(TMEM_COLS * CTAS_PER_SM <= 512, "tensor memory holds 512 columns per SM");
};

// One tile of work: (weight-row tile, token tile).  Tiles are numbered in bands of TILE_BAND token
// tiles: inside a band the token tile runs fastest, then the weight-row tile, so the CTAs that run
// side by side share both a few weight slabs and a few activation tiles through the L2 (prompts:
// an expert has several token tiles, and every activation tile meets every weight-row tile).  A
// CTA (or pair) takes tiles w, w + workers, ...; a pair's weight-row tile is two adjacent ones.
struct TileInfo { int expert, row0, count, mx; };
constexpr int TILE_BAND = 8;

__device__ __forceinline__ TileInfo tile_info(int id, int n_ty, int n_mx, int bn, const int* tile_expert,
                                              const int* tile_row0, const int* tile_count, int R) {
    TileInfo t;
    const int full = (n_ty / TILE_BAND) * TILE_BAND;          // token tiles in whole bands
    int ty;
    if (id < full * n_mx) {
        const int band = id / (TILE_BAND * n_mx), rem = id - band * (TILE_BAND * n_mx);
        t.mx = rem / TILE_BAND;
        ty = band * TILE_BAND + rem % TILE_BAND;
    } else {
        const int rem = id - full * n_mx, w = n_ty - full;    // the last, narrower band
        t.mx = rem / w;
        ty = full + rem % w;
    }
    if (tile_expert) {
        t.expert = tile_expert[ty];
        t.row0 = tile_row0[ty];
        t.count = tile_count[ty];
    } else {
        t.expert = 0;
        t.row0 = ty * bn;
        t.count = min(bn, R - t.row0);
    }
    return t;
}

// A second product in the same launch: one group, token tiles of BN consecutive rows, its own operands, output and
// sizes.  The persistent CTAs walk the tiles of both products in one interleaved sequence, so that a product bound by
// the tensor cores (a prompt's shared expert: every weight block is reused by all token tiles out of the L2) runs
// on some SMs while a product bound by its weight stream (the prompt's routed experts: every block read once from
// DRAM) runs on the others, and each SM alternates between the two; as two launches one would wait for the other,
// since either fills the GPU with one CTA per SM.
struct NoSecond {};
struct Second {
    CUtensorMap map_w, map_x, map_x_tail;
    void* out;
    int R, N, K;
    int first;          // 0: the second product's tiles are spread evenly among the first's; 1: they all come first
};

// Which product and which of its tiles the u-th unit of work is: the second product's total2 tiles are spread evenly
// over the total1 + total2 units (unit u is its c-th tile iff the count c = floor(u * total2 / all) grows at u + 1).
struct Unit { int second, id; };
__device__ __forceinline__ Unit unit_of(int u, int total1, int total2, int second_first) {
    Unit w;
    if (second_first) {
        w.second = u < total2 ? 1 : 0;
        w.id = w.second ? u : u - total2;
        return w;
    }
    const long long all = (long long)total1 + total2;
    const int c = (int)((long long)u * total2 / all), c_next = (int)((long long)(u + 1) * total2 / all);
    w.second = c_next > c ? 1 : 0;
    w.id = w.second ? c : u - c;
    return w;
}

// KSPLIT: the instantiation whose units of work are shares of a tile's K (see k_splits below); the others walk whole
// tiles and carry none of that arithmetic in their loops.  SECOND = Second: the instantiation that walks two products.
template <int BN, bool SWIGLU, typename TO, bool PAIR, bool KSPLIT, typename SECOND>
__global__ void __launch_bounds__((Tile<BN, PAIR>::THREADS), (Tile<BN, PAIR>::CTAS_PER_SM))
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_x_tail, TO* __restrict__ out,
               const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
               const int* __restrict__ tile_count, const int* __restrict__ n_tiles, int R, int N, int K,
               int stream_weights, int* __restrict__ status, int k_splits, const __grid_constant__ SECOND second) {
    // Bit 1 of stream_weights: the weights, the tile list and the sizes were final before the kernel ahead of this
    // one in the stream started (a down projection behind its gate/up product; a product with one group), so the
    // thread that streams the weights does not wait for that kernel: its loads are in flight while the kernel ahead
    // still runs.  Everything else (the token rows above all) waits as usual.
    const bool early_weights = (stream_weights & 2) != 0;
    if (!early_weights) tq_grid_wait();      // everything below may read what the previous kernel wrote
    using T = Tile<BN, PAIR>;
    constexpr bool DUAL = !std::is_same<SECOND, NoSecond>::value;
    static_assert(!(DUAL && KSPLIT), "a launch either walks two products or shares K out");
    constexpr int COLS = SWIGLU ? BM / 2 : BM;         // output columns of a weight-row tile
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem_base;

    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;                 // place in the pair; 0 issues the products
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int n_ty = tile_expert ? n_tiles[0] : (R + BN - 1) / BN;       // token tiles
    const int n_m1 = (N + COLS - 1) / COLS;                              // weight-row tiles
    const int n_mx = PAIR ? (n_m1 + 1) / 2 : n_m1;                       // ... as units of work
    const int total = n_ty * n_mx;
    // k_splits > 1: a tile's k-blocks are shared out over that many units of work, each writing its partial sums to
    // a slice of its own of `out` ([k_splits][R][N]; the caller adds the slices up in order).  For products with few
    // tiles and a long K (a down projection of a few tokens), which would otherwise keep a few SMs busy for long.
    // the second product's sizes (DUAL only; the rest of the code reads them through `if constexpr`)
    int R2 = 0, N2 = 0, n_ty2 = 0, n_m1_2 = 0, n_mx2 = 0, total2 = 0, num_kb2 = 0, second_first = 0;
    if constexpr (DUAL) {
        R2 = second.R; N2 = second.N; second_first = second.first;
        n_ty2 = (R2 + BN - 1) / BN;
        n_m1_2 = (N2 + COLS - 1) / COLS;
        n_mx2 = PAIR ? (n_m1_2 + 1) / 2 : n_m1_2;
        total2 = n_ty2 * n_mx2;
        num_kb2 = (second.K + BK - 1) / BK;
    }
    const int units = KSPLIT ? total * k_splits : (DUAL ? total + total2 : total);
    if (worker >= units) return;                                         // both CTAs of a pair leave together
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int kb_per = KSPLIT ? (num_kb + k_splits - 1) / k_splits : num_kb;   // the host made sure every share holds a block

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;     // swizzled tiles want 1024-byte alignment
    constexpr int SA = T::A_SLOTS, SB = T::B_SLOTS;
    // One pair of barriers per k-block in flight (SA of them): `full` hears of the weight block and of the
    // token block (two arrivals and their bytes), `done` of the products that read them.  Block i uses weight
    // slot i % SA and token slot i % SB.
    const uint32_t bars = base + SA * T::A_BYTES + SB * T::B_BYTES;  // full[SA], done[SA], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto done_bar = [&](int s) { return bars + 8u * (SA + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * SA + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * SA + 2 + b); };
    auto a_tile = [&](int s) { return base + s * T::A_BYTES; };
    auto b_tile = [&](int s) { return base + SA * T::A_BYTES + s * T::B_BYTES; };

    if (threadIdx.x == 0) {
        s_abort = 0;
        // pairs: the stage barriers that count bytes (of both CTAs' loads) and the accumulator-drained barriers
        // live in the first CTA; the others are signalled in both CTAs at once by the products' commits
        for (int s = 0; s < SA; ++s) { mbar_init(full_bar(s), 2); mbar_init(done_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), (PAIR ? 2 : 1) * T::EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&s_tmem_base)), "r"((uint32_t)T::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(&s_tmem_base)), "r"((uint32_t)T::TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (PAIR) cluster_sync_all(); else __syncthreads();     // barriers are ready in both CTAs before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // only now: a dependent kernel that took tensor memory first could starve a CTA of this grid that
    // had not allocated yet, and then wait forever for this grid to finish
    tq_grid_launch_dependents();
    const uint32_t tmem_base = s_tmem_base;
    if (early_weights && warp != 0) tq_grid_wait();

    // The two producers are one thread each and their loops are kept to a few instructions per block: a single
    // thread runs one dependent instruction every few cycles, and a block lasts only some hundred cycles.
    if (warp == 0) {
        // ---------------- weight blocks: one stream of k-blocks across all of this CTA's tiles ----------------
        if (lane == 0) {
            // weights that only one token tile reads (a decode step, a short prompt) are streamed: first to leave
            // the L2; weights that several token tiles share stay
            const uint64_t policy = (stream_weights & 1) ? policy_evict_first() : policy_evict_last();
            const uint64_t keep = policy_evict_last();
            (void)keep;
            int slot = 0, issued = 0;
            uint32_t phase = 0;      // parity of the slot's current use
            bool ok = true;
            for (int u = worker; u < units && ok; u += workers) {
                int id = KSPLIT ? u % total : u, kb0 = KSPLIT ? (u / total) * kb_per : 0, kb1 = KSPLIT ? min(num_kb, kb0 + kb_per) : num_kb;
                bool is2 = false;                  // a tile of the second product
                if constexpr (DUAL) {
                    const Unit w = unit_of(u, total, total2, second_first);
                    is2 = w.second != 0;
                    id = w.id;
                    if (is2) kb1 = num_kb2;
                }
                const TileInfo t = is2 ? tile_info(id, n_ty2, n_mx2, BN, nullptr, nullptr, nullptr, R2)
                                       : tile_info(id, n_ty, n_mx, BN, tile_expert, tile_row0, tile_count, R);
                const int wt = t.expert * (is2 ? n_m1_2 : n_m1) + (PAIR ? 2 * t.mx + (int)rank : t.mx);    // packed weight tile
                const CUtensorMap* mw = &map_w;
                uint64_t pol = policy;
                if constexpr (DUAL) if (is2) { mw = &second.map_w; pol = n_ty2 > 1 ? keep : policy_evict_first(); }
                for (int kb = kb0; kb < kb1; ++kb) {
                    // the slot is free once the products of the block SA before this one are done
                    if (!mbar_wait(done_bar(slot), phase ^ 1u, &s_abort)) { ok = false; break; }
                    if (PAIR) {
                        // the first CTA expects the bytes of both (the halves are equal); the second only loads
                        if (rank == 0) mbar_expect_tx(full_bar(slot), 2u * T::A_BYTES);
                        tma_load_block_pair(a_tile(slot), mw, kb, wt, rank == 0 ? full_bar(slot) : map_to_cta(full_bar(slot), 0), pol);
                    } else {
                        mbar_expect_tx(full_bar(slot), (uint32_t)T::A_BYTES);
                        tma_load_block(a_tile(slot), mw, kb, wt, full_bar(slot), pol);
                    }
                    ++issued;
                    if (++slot == SA) { slot = 0; phase ^= 1u; }
                }
            }
            if (s_abort && rank == 0) {
                // wait (bounded) for the copies this thread started, so none lands after the CTA is gone
                // (a block whose token half was never issued stays incomplete: that wait runs out)
                for (int j = issued > SA ? issued - SA : 0; j < issued; ++j)
                    for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(full_bar(j % SA), (uint32_t)(j / SA) & 1u); ++i) {}
            }
        }
    } else if (warp == 2) {
        // ---------------- token blocks: block i goes to token slot i % SB and reports to full[i % SA] ----------------
        if (lane == 0) {
            const uint64_t policy = policy_evict_last();
            int slot = 0, fb = 0, issued = 0;
            int freed = 0;           // done[] index of the block SB before this one ...
            uint32_t freed_phase = 0;   // ... and the parity of that block's use of it
            bool ok = true;
            for (int u = worker; u < units && ok; u += workers) {
                int id = KSPLIT ? u % total : u, kb0 = KSPLIT ? (u / total) * kb_per : 0, kb1 = KSPLIT ? min(num_kb, kb0 + kb_per) : num_kb;
                bool is2 = false;                  // a tile of the second product
                if constexpr (DUAL) {
                    const Unit w = unit_of(u, total, total2, second_first);
                    is2 = w.second != 0;
                    id = w.id;
                    if (is2) kb1 = num_kb2;
                }
                const TileInfo t = is2 ? tile_info(id, n_ty2, n_mx2, BN, nullptr, nullptr, nullptr, R2)
                                       : tile_info(id, n_ty, n_mx, BN, tile_expert, tile_row0, tile_count, R);
                const int n_mma = (t.count + 15) & ~15;                                   // N of the products
                const int rows = PAIR ? n_mma / 2 : t.count;                              // token rows this CTA loads ...
                const int row0 = t.row0 + (PAIR ? (int)rank * (n_mma / 2) : 0);           // ... from here
                const int boxes = rows / T::BOX_ROWS;
                const int tails = (rows - boxes * T::BOX_ROWS + T::TAIL_ROWS - 1) / T::TAIL_ROWS;
                const uint32_t bytes = (uint32_t)(boxes * T::BOX_BYTES + tails * T::TAIL_BYTES);
                const CUtensorMap* mx = &map_x;
                const CUtensorMap* mxt = &map_x_tail;
                if constexpr (DUAL) if (is2) { mx = &second.map_x; mxt = &second.map_x_tail; }
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (issued >= SB) {
                        if (!mbar_wait(done_bar(freed), freed_phase, &s_abort)) { ok = false; break; }
                        if (++freed == SA) { freed = 0; freed_phase ^= 1u; }
                    }
                    const uint32_t dst = b_tile(slot);
                    if (PAIR) {
                        const uint32_t bar = rank == 0 ? full_bar(fb) : map_to_cta(full_bar(fb), 0);
                        if (rank == 0) mbar_expect_tx(full_bar(fb), 2u * bytes);
                        for (int bx = 0; bx < boxes; ++bx)
                            tma_load_2d_pair(dst + bx * T::BOX_BYTES, mx, kb * BK, row0 + bx * T::BOX_ROWS, bar, policy);
                        for (int bx = 0; bx < tails; ++bx)
                            tma_load_2d_pair(dst + boxes * T::BOX_BYTES + bx * T::TAIL_BYTES, mxt, kb * BK,
                                             row0 + boxes * T::BOX_ROWS + bx * T::TAIL_ROWS, bar, policy);
                    } else {
                        mbar_expect_tx(full_bar(fb), bytes);
                        for (int bx = 0; bx < boxes; ++bx)
                            tma_load_2d(dst + bx * T::BOX_BYTES, mx, kb * BK, row0 + bx * T::BOX_ROWS, full_bar(fb), policy);
                        for (int bx = 0; bx < tails; ++bx)
                            tma_load_2d(dst + boxes * T::BOX_BYTES + bx * T::TAIL_BYTES, mxt, kb * BK,
                                        row0 + boxes * T::BOX_ROWS + bx * T::TAIL_ROWS, full_bar(fb), policy);
                    }
                    ++issued;
                    if (++slot == SB) slot = 0;
                    if (++fb == SA) fb = 0;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (the pair's first CTA issues for both) ----------------
        if (lane == 0 && rank == 0) {
            int sa = 0, sb = 0, it = 0;      // weight slot (and barrier) and token slot of the next block
            uint32_t phase = 0;
            bool ok = true;
            for (int u = worker; u < units && ok; u += workers, ++it) {
                int id = KSPLIT ? u % total : u, kb0 = KSPLIT ? (u / total) * kb_per : 0, kb1 = KSPLIT ? min(num_kb, kb0 + kb_per) : num_kb;
                bool is2 = false;                  // a tile of the second product
                if constexpr (DUAL) {
                    const Unit w = unit_of(u, total, total2, second_first);
                    is2 = w.second != 0;
                    id = w.id;
                    if (is2) kb1 = num_kb2;
                }
                const TileInfo t = is2 ? tile_info(id, n_ty2, n_mx2, BN, nullptr, nullptr, nullptr, R2)
                                       : tile_info(id, n_ty, n_mx, BN, tile_expert, tile_row0, tile_count, R);
                // N of the products: this tile's rows; pairs: M = 256, 128 weight rows from each CTA
                const uint32_t idesc = umma_idesc((t.count + 15) & ~15) + (PAIR ? ((uint32_t)(BM >> 4) << 24) : 0u);
                const int b = it & 1;
                const uint32_t acc = tmem_base + (uint32_t)(b * T::ACC_COLS);
                // the epilogue must have drained this accumulator (two tiles ago)
                if (it >= 2) ok = mbar_wait(acc_empty(b), (uint32_t)((it >> 1) - 1) & 1u, &s_abort);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = kb0; kb < kb1; ++kb) {
                    ok = mbar_wait(full_bar(sa), phase, &s_abort);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                        const uint64_t ad = umma_desc(a_tile(sa) + k * UMMA_K * 2), bd = umma_desc(b_tile(sb) + k * UMMA_K * 2);
                        if (PAIR) umma_pair(acc, ad, bd, idesc, accum); else umma(acc, ad, bd, idesc, accum);
                    }
                    // the slots are free (in both CTAs) once these MMAs have read them
                    if (PAIR) umma_commit_pair(done_bar(sa)); else umma_commit(done_bar(sa));
                    if (++sa == SA) { sa = 0; phase ^= 1u; }
                    if (++sb == SB) sb = 0;
                }
                // this tile's accumulator is complete once all MMAs are done
                if (ok) { if (PAIR) umma_commit_pair(acc_full(b)); else umma_commit(acc_full(b)); }
            }
        }
    } else {
        // ---------------- epilogue: warps 3.., TMEM lane quarter = warp % 4 ----------------
        const int quarter = warp & 3;
        const int group0 = (warp - 3) >> 2;                // wide tiles: which groups of 16 token rows (even or odd)
        constexpr int GROUP_STEP = T::EPI_WARPS / 4;
        // plain: lane = weight row = output column.  SwiGLU: lanes 0..15 hold the gate of 16 columns, lanes
        // 16..31 the up of the same columns; after the exchange the low half writes token rows 0..7 of each
        // group of 16 and the high half rows 8..15.
        const bool high = SWIGLU && lane >= 16;
        const int r = SWIGLU ? quarter * 16 + (lane & 15) : quarter * 32 + lane;     // output column within the tile
        int it = 0;
        bool ok = true;
        for (int u = worker; u < units && ok; u += workers, ++it) {
            int id = KSPLIT ? u % total : u, kb0 = KSPLIT ? (u / total) * kb_per : 0, kb1 = KSPLIT ? min(num_kb, kb0 + kb_per) : num_kb;
            bool is2 = false;                  // a tile of the second product
            if constexpr (DUAL) {
                const Unit w = unit_of(u, total, total2, second_first);
                is2 = w.second != 0;
                id = w.id;
                if (is2) kb1 = num_kb2;
            }
            const TileInfo t = is2 ? tile_info(id, n_ty2, n_mx2, BN, nullptr, nullptr, nullptr, R2)
                                   : tile_info(id, n_ty, n_mx, BN, tile_expert, tile_row0, tile_count, R);
            const int b = it & 1;
            const int n = (PAIR ? 2 * t.mx + (int)rank : t.mx) * COLS + r;           // output column
            TO* out_u = KSPLIT ? out + (size_t)(u / total) * R * N : out;            // this share's slice (kb0, kb1 unused here)
            int Nn = N;                                                              // width of this product's output
            if constexpr (DUAL) if (is2) { out_u = (TO*)second.out; Nn = N2; }
            (void)kb0; (void)kb1;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full(b), (uint32_t)(it >> 1) & 1u, &s_abort));   // warp-uniform
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem_base + (uint32_t)(b * T::ACC_COLS) + ((uint32_t)(quarter * 32) << 16);
            uint32_t buf[2][16];                           // the loop is unrolled: both are registers
            if (group0 * 16 < t.count) tmem_ld16(lane_addr + group0 * 16, buf[0]);
#pragma unroll
            for (int i = 0; i < BN / (16 * GROUP_STEP); ++i) {
                const int c0 = (group0 + i * GROUP_STEP) * 16;
                if (c0 >= t.count) break;                  // uniform across the warp
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t (&g)[16] = buf[i & 1];
                const int c_next = c0 + 16 * GROUP_STEP;   // the next group is on its way while this one is written out
                if (i + 1 < BN / (16 * GROUP_STEP) && c_next < t.count) tmem_ld16(lane_addr + c_next, buf[(i + 1) & 1]);
                if (SWIGLU) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // low lanes keep rows 0..7 and send their gate of rows 8..15; high lanes the other way round
                        const uint32_t got = __shfl_xor_sync(0xffffffffu, high ? g[j] : g[8 + j], 16);
                        const float gate = __uint_as_float(high ? got : g[j]);
                        const float up = __uint_as_float(high ? g[8 + j] : got);
                        const int c = c0 + j + (high ? 8 : 0);
                        if (n < Nn && c < t.count) out_u[(size_t)(t.row0 + c) * Nn + n] = tq_from_float<TO>(silu_mul<TO>(gate, up));
                    }
                } else if (n < Nn) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < t.count) out_u[(size_t)(t.row0 + c0 + j) * Nn + n] = tq_from_float<TO>(__uint_as_float(g[j]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {                               // this warp has read its part of the accumulator
                if (PAIR) mbar_arrive_cluster(map_to_cta(acc_empty(b), 0)); else mbar_arrive(acc_empty(b));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    // pairs: neither CTA may leave (or free tensor memory) while the other can still signal it or read through it
    if (PAIR) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && s_abort) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
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

// activations: bf16 matrix [rows][K] row-major; box [box_rows][64], 128-byte swizzle
int make_map_x(CUtensorMap* map, const void* ptr, uint64_t k, uint64_t rows, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) TQ_FAIL(-3, "gemm_tc: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {k, rows};
    cuuint64_t strides[1] = {k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TQ_FAIL(-3, "gemm_tc: cuTensorMapEncodeTiled (activations) failed with code %d", (int)r);
    return 0;
}

// packed weights: [tiles][k-blocks][128 rows][64 elements], every [128 x 64] block contiguous (16 KiB)
int make_map_w(CUtensorMap* map, const void* ptr, uint64_t k_blocks, uint64_t tiles) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) TQ_FAIL(-3, "gemm_tc: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)BK, (cuuint64_t)BM, k_blocks, tiles};
    cuuint64_t strides[3] = {(cuuint64_t)BK * 2, (cuuint64_t)BK * BM * 2, k_blocks * BK * BM * 2};
    cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)BM, 1, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TQ_FAIL(-3, "gemm_tc: cuTensorMapEncodeTiled (weights) failed with code %d", (int)r);
    return 0;
}

template <int BN, bool SWIGLU, typename TO, bool PAIR, bool KSPLIT = false, typename SECOND = NoSecond>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mxt, void* out, const int* te, const int* tr,
           const int* tc, const int* nt, int grid_y, int R, int N, int K, int G, int* status, int sm_share_pct,
           int k_splits, cudaStream_t stream, const SECOND& second = SECOND(), long long tiles2 = 0, int early_weights = 0) {
    using T = Tile<BN, PAIR>;
    auto kern = gemm_tc_kernel<BN, SWIGLU, TO, PAIR, KSPLIT, SECOND>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess) TQ_FAIL(-1, "gemm_tc: cannot reserve %d bytes of shared memory: %s", T::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    // persistent CTAs (or pairs): at most what the GPU runs at once; each walks tiles w, w + workers, ...
    static int resident = 0;
    if (resident == 0) {
        int dev = 0, n_sm = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
        resident = n_sm * T::CTAS_PER_SM;
        if (PAIR) {
            // pairs share a cluster of two SMs; the GPU may not pair up every SM
            cudaLaunchConfig_t cfg;
            cudaLaunchAttribute attr[2];
            tq_launch(n_sm & ~1, T::THREADS, T::SMEM_BYTES, stream, 2).config(cfg, attr);
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) == cudaSuccess && clusters > 0) resident = 2 * clusters;
            else { cudaGetLastError(); resident = (n_sm / 2) & ~1; }
            if (getenv("TQ_DEBUG")) fprintf(stderr, "gemm_tc pair BN=%d: clusters=%d resident=%d\n", BN, clusters, resident);
        }
    }
    constexpr int COLS = SWIGLU ? BM / 2 : BM;
    const long long n_m1 = (N + COLS - 1) / COLS;
    const long long tiles = (PAIR ? (n_m1 + 1) / 2 : n_m1) * grid_y * k_splits + tiles2;      // units of work
    const long long want = PAIR ? 2 * tiles : tiles;
    // sm_share_pct in 1..99: this launch takes only that share of the CTAs the GPU runs at once, so that another
    // launch on another stream runs beside it instead of behind it (a compute-bound product beside a memory-bound one)
    long long room = resident;
    if (sm_share_pct > 0 && sm_share_pct < 100) {
        room = (long long)resident * sm_share_pct / 100;
        if (PAIR) room &= ~1LL;
        if (room < (PAIR ? 2 : 1)) room = PAIR ? 2 : 1;
    }
    const int grid = (int)(want < room ? want : room);
    tq_launch(grid, T::THREADS, T::SMEM_BYTES, stream, PAIR ? 2 : 1)(kern, mw, mx, mxt, (TO*)out, te, tr, tc, nt, R, N, K,
        /* stream_weights: on average at most one token tile per group */ ((te != nullptr && (long long)R <= (long long)G * BN) ? 1 : 0) | (early_weights ? 2 : 0), status,
        k_splits, second);
    TQ_CHECK_LAUNCH("gemm_tc");
    return 0;
}

}  // namespace

// X [R, K] bf16; W: the [G, Nw, K] weights (Nw = N, or 2N with swiglu: gate rows then up rows) PACKED into
// [G * tiles][ceil(K/64)][128][64] blocks, zero-padded, where tiles = ceil(N/128) (plain) or ceil(N/64)
// (swiglu: a block's rows 32q+i are the gate and 32q+16+i the up of column 64*tile+16q+i, i < 16);
// out [R, N] in bf16 or fp32.
// tile_* describe token tiles of at most `bn` rows that never span two groups (null: one group, tiles
// of bn consecutive rows).  pair: token tiles of 128 or 256 rows run on pairs of CTAs (cta_group::2: each
// CTA holds 128 weight rows and half of the token rows).  status: one int in device memory, set to 1 if
// a bounded wait ran out.  sm_share_pct: 0 or 100 = the launch may fill the GPU; 1..99 = it takes that share of the
// CTAs the GPU runs at once.  k_splits > 1 (plain products, fp32 out): out is [k_splits][R][N], slice s holding the
// partial sums over the s-th share of K; the caller adds them up.  early_weights: the caller vouches that W, the
// tile arrays and n_tiles were final before the kernel ahead of this one in the stream started; the weight stream then
// starts without waiting for that kernel (programmatic dependent launch), the token rows wait for it as always.
TQ_EXPORT int tq_gemm_tc(const void* X, const void* W, void* out, int out_dtype, const int* tile_expert,
                         const int* tile_row0, const int* tile_count, const int* n_tiles, int max_tiles, int bn,
                         int R, int N, int K, int G, int swiglu, int pair, int* status, int sm_share_pct,
                         int k_splits, int early_weights, cudaStream_t stream) {
    if (R == 0 || (tile_expert && max_tiles == 0)) return 0;
    TQ_REQUIRE(k_splits >= 1, "gemm_tc: %d shares of K", k_splits);
    if (k_splits > 1) {
        TQ_REQUIRE(!swiglu && out_dtype == TQ_F32, "gemm_tc: K is shared out only for plain products with float32 partial sums");
        const int num_kb = (K + BK - 1) / BK, per = (num_kb + k_splits - 1) / k_splits;
        TQ_REQUIRE((k_splits - 1) * per < num_kb, "gemm_tc: %d shares of %d k-blocks would leave a share empty", k_splits, num_kb);
    }
    TQ_REQUIRE(R > 0 && N > 0 && K > 0 && G > 0, "gemm_tc: bad sizes R=%d N=%d K=%d G=%d", R, N, K, G);
    TQ_REQUIRE(K % 8 == 0, "gemm_tc: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    TQ_REQUIRE(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
    TQ_REQUIRE(bn == 16 || bn == 32 || bn == 64 || bn == 128 || bn == 256, "gemm_tc: token tile %d is not one of 16, 32, 64, 128, 256", bn);
    TQ_REQUIRE(!pair || bn >= 128, "gemm_tc: pairs of CTAs take token tiles of 128 or 256 rows, not %d", bn);
    TQ_REQUIRE(status != nullptr, "gemm_tc: a status word is required");
    TQ_REQUIRE(out_dtype == TQ_BF16 || out_dtype == TQ_F32, "gemm_tc: unknown output type %d", out_dtype);
    const int grid_y = tile_expert ? max_tiles : (R + bn - 1) / bn;
    CUtensorMap mw, mx, mxt;
    const int n_mx = swiglu ? (N + BM / 2 - 1) / (BM / 2) : (N + BM - 1) / BM;
    int rc = make_map_w(&mw, W, (uint64_t)((K + BK - 1) / BK), (uint64_t)G * n_mx);
    if (rc) return rc;
    rc = make_map_x(&mx, X, (uint64_t)K, (uint64_t)R, (uint32_t)(bn < 64 ? bn : 64));
    if (rc) return rc;
    rc = make_map_x(&mxt, X, (uint64_t)K, (uint64_t)R, 16u);
    if (rc) return rc;
#define TC_ARGS mw, mx, mxt, out, tile_expert, tile_row0, tile_count, n_tiles, grid_y, R, N, K, G, status, sm_share_pct, k_splits, stream, NoSecond(), 0, early_weights
#define TC_CASE(BN_, PAIR_)                                                                          \
    if (bn == BN_ && (pair != 0) == PAIR_) {                                                         \
        if (swiglu) {                                                                                \
            if (out_dtype == TQ_BF16) return launch<BN_, true, __nv_bfloat16, PAIR_>(TC_ARGS);        \
            return launch<BN_, true, float, PAIR_>(TC_ARGS);                                          \
        }                                                                                            \
        if (out_dtype == TQ_BF16) return launch<BN_, false, __nv_bfloat16, PAIR_>(TC_ARGS);           \
        return launch<BN_, false, float, PAIR_>(TC_ARGS);                                             \
    }
    if (k_splits > 1) {          // plain, float32 partial sums (checked above); narrow token tiles on single CTAs
        TQ_REQUIRE(!pair && bn <= 64, "gemm_tc: K is shared out for token tiles of 16, 32 or 64 rows on single CTAs, not %d%s", bn, pair ? " on pairs" : "");
        if (bn == 16) return launch<16, false, float, false, true>(TC_ARGS);
        if (bn == 32) return launch<32, false, float, false, true>(TC_ARGS);
        return launch<64, false, float, false, true>(TC_ARGS);
    }
    TC_CASE(16, false) TC_CASE(32, false) TC_CASE(64, false) TC_CASE(128, false) TC_CASE(256, false)
    TC_CASE(128, true) TC_CASE(256, true)
#undef TC_CASE
#undef TC_ARGS
    TQ_FAIL(-2, "gemm_tc: unreachable");
}

// Two products in one launch: the first as tq_gemm_tc computes it over the layout's groups (X, W, out, tile_*; G
// groups), the second over one group with token tiles of `bn` consecutive rows (X2 [R2, K2], W2 packed for N2 x K2,
// out2 [R2, N2]).  Both are plain or both SwiGLU, with the same output type; SwiGLU writes bf16 and a plain product
// float32 (the experts' two steps); CTA pairs with token tiles of 128 or 256 rows.  second_first: 0 = the second
// product's tiles are spread evenly among the first's, 1 = they come first.
TQ_EXPORT int tq_gemm_tc_dual(const void* X, const void* W, void* out, const int* tile_expert, const int* tile_row0,
                              const int* tile_count, const int* n_tiles, int max_tiles, int R, int N, int K, int G,
                              const void* X2, const void* W2, void* out2, int R2, int N2, int K2, int out_dtype,
                              int bn, int swiglu, int* status, int second_first, cudaStream_t stream) {
    TQ_REQUIRE(tile_expert && tile_row0 && tile_count && n_tiles, "gemm_tc_dual: the first product needs a layout");
    TQ_REQUIRE(R > 0 && N > 0 && K > 0 && G > 0 && R2 > 0 && N2 > 0 && K2 > 0, "gemm_tc_dual: bad sizes R=%d N=%d K=%d G=%d, R2=%d N2=%d K2=%d", R, N, K, G, R2, N2, K2);
    TQ_REQUIRE(K % 8 == 0 && K2 % 8 == 0, "gemm_tc_dual: K=%d and K2=%d must be multiples of 8 (16-byte rows for TMA)", K, K2);
    TQ_REQUIRE(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)X2 % 16) == 0 && ((uintptr_t)W2 % 16) == 0,
               "gemm_tc_dual: operands must be 16-byte aligned");
    TQ_REQUIRE(bn == 128 || bn == 256, "gemm_tc_dual: token tiles of 128 or 256 rows (pairs of CTAs), not %d", bn);
    TQ_REQUIRE((swiglu && out_dtype == TQ_BF16) || (!swiglu && out_dtype == TQ_F32),
               "gemm_tc_dual: SwiGLU products write bfloat16 and plain products float32 (got swiglu=%d, type %d)", swiglu, out_dtype);
    TQ_REQUIRE(status != nullptr, "gemm_tc_dual: a status word is required");
    if (max_tiles == 0) return tq_gemm_tc(X2, W2, out2, out_dtype, nullptr, nullptr, nullptr, nullptr, 0, bn, R2, N2, K2, 1, swiglu, 1, status, 0, 1, 0, stream);
    const int cols = swiglu ? BM / 2 : BM;
    const int n_m1 = (N + cols - 1) / cols, n_m1_2 = (N2 + cols - 1) / cols;
    CUtensorMap mw, mx, mxt;
    Second sec;
    int rc = make_map_w(&mw, W, (uint64_t)((K + BK - 1) / BK), (uint64_t)G * n_m1);
    if (rc) return rc;
    if ((rc = make_map_x(&mx, X, (uint64_t)K, (uint64_t)R, 64u))) return rc;
    if ((rc = make_map_x(&mxt, X, (uint64_t)K, (uint64_t)R, 16u))) return rc;
    if ((rc = make_map_w(&sec.map_w, W2, (uint64_t)((K2 + BK - 1) / BK), (uint64_t)n_m1_2))) return rc;
    if ((rc = make_map_x(&sec.map_x, X2, (uint64_t)K2, (uint64_t)R2, 64u))) return rc;
    if ((rc = make_map_x(&sec.map_x_tail, X2, (uint64_t)K2, (uint64_t)R2, 16u))) return rc;
    sec.out = out2; sec.R = R2; sec.N = N2; sec.K = K2; sec.first = second_first ? 1 : 0;
    const long long tiles2 = (long long)((n_m1_2 + 1) / 2) * ((R2 + bn - 1) / bn);
#define TC_DUAL(BN_)                                                                                                       \
    if (bn == BN_) {                                                                                                       \
        if (swiglu) return launch<BN_, true, __nv_bfloat16, true, false, Second>(mw, mx, mxt, out, tile_expert, tile_row0, \
            tile_count, n_tiles, max_tiles, R, N, K, G, status, 0, 1, stream, sec, tiles2);                                \
        return launch<BN_, false, float, true, false, Second>(mw, mx, mxt, out, tile_expert, tile_row0, tile_count,        \
            n_tiles, max_tiles, R, N, K, G, status, 0, 1, stream, sec, tiles2);                                            \
    }
    TC_DUAL(128) TC_DUAL(256)
#undef TC_DUAL
    TQ_FAIL(-2, "gemm_tc_dual: unreachable");
}
