// Mixture-of-experts feed-forward: router, expert-sorted row layout, exact grouped GEMM, combine.
//
//   tq_router_topk    logits = Wr x (fp32), softmax over all experts, k largest (ties to the lowest
//                     index), optional renormalisation; the shared expert's sigmoid gate in the
//                     same pass
//   tq_router_select  the selection alone, from logits that a tensor-core product left (prompts)
//   tq_moe_align      stable counting sort of (token, choice) pairs by expert, and the list of row
//                     tiles the grouped GEMMs walk
//   tq_router_small   decode steps: logits, selection, layout, tile list and the expert-sorted copies
//                     of the token rows in one launch
//   tq_grouped_gemm   C[rows of expert e] = A[rows] W[e]^T, fp32 accumulation on CUDA cores (the
//                     exact path; any sizes), optionally with SiLU(gate)*up fused in
//   tq_moe_combine    y[t] = sum_j w[t,j] Y[row(t,j)] + s[t] Y_shared[t], in the order chosen
//
// Formulas as the reference computes them on the CPU (src/engine/tq_moe.c): router logits
// :612-618; selection of k experts :630-646 (the reference takes a softmax over the k picked
// logits :659-678, which is the renormalised case here, and breaks exact ties toward the highest
// index); experts g = Wg x, u = Wu x, h = silu(g)*u, o = Wd h, out += w*o :975-999 (exact exp
// here, a fast approximation there :42-92); shared expert scaled by sigmoid(w_sg . x) :1006-1058;
// accumulation order: chosen experts first, shared expert last.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define ROUTER_MAX_EXPERTS 4096
#define ROUTER_MAX_STAGED_H 12288     // widths up to this are staged in shared memory as fp32 (48 KiB)

// ---------------------------------------------------------------------------------------
// Router: one block per token.  The token's row is staged in shared memory as fp32; each warp
// takes whole rows of the router matrix (and the shared expert's gate row) and reads them with
// 16-byte loads, eight elements per lane per step, in a fixed order; warp 0 then does the softmax
// and the selection.
// ---------------------------------------------------------------------------------------
// 16 bytes from global memory with an L2 eviction policy (createpolicy): the router's matrix is a few hundred KB
// that every step reads again; marked evict-last it stays in the L2 while the experts' weights stream through.
__device__ __forceinline__ uint4 ld_global_policy(const void* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.L2::cache_hint.v4.b32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    return v;
}

template <typename TW> struct RowVec { };
template <> struct RowVec<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ void load_keep(const __nv_bfloat16* p, float (&f)[8], uint64_t policy) {
        const uint4 v = ld_global_policy(p, policy);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint4 v;
        uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); u[i] = *reinterpret_cast<const uint32_t*>(&h); }
        *reinterpret_cast<uint4*>(p) = v;
    }
};
template <> struct RowVec<float> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void load_keep(const float* p, float (&f)[8], uint64_t policy) {
        const uint4 a = ld_global_policy(p, policy), b = ld_global_policy(p + 4, policy);
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// Kernel 1: logits[t, e] = x[t] . w[e] for a chunk of rows (grid: tokens x row chunks).
template <typename TA, typename TW, bool STAGED>
__global__ void router_logits_kernel(const TA* __restrict__ x, const TW* __restrict__ wr, const TW* __restrict__ wsg,
                                     float* __restrict__ logits, int H, int E, int rows_per_cta, int vec_ok) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ float s_x[];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const TA* xr = x + (size_t)t * H;
    const int rows = E + (wsg ? 1 : 0);
    if (STAGED) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) s_x[i] = tq_to_float(xr[i]);
        __syncthreads();
    }
    const int Hv = vec_ok ? (H / 8) * 8 : 0;    // part of the row read with 16-byte loads
    const int e0 = blockIdx.y * rows_per_cta, e1 = min(rows, e0 + rows_per_cta);
    for (int e = e0 + warp; e < e1; e += nwarps) {
        const TW* w = e < E ? wr + (size_t)e * H : wsg;
        float s = 0.f;
#pragma unroll 4
        for (int i = lane * 8; i < Hv; i += 256) {          // unrolled: four 16-byte loads in flight per lane
            float f[8];
            RowVec<TW>::load(w + i, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) s = fmaf(STAGED ? s_x[i + j] : tq_to_float(xr[i + j]), f[j], s);
        }
        for (int i = Hv + lane; i < H; i += 32) s = fmaf(STAGED ? s_x[i] : tq_to_float(xr[i]), tq_to_float(w[i]), s);
        s = tq_warp_sum(s);
        if (lane == 0) logits[(size_t)t * (E + 1) + e] = s;
    }
}

// Floats compare like these integers (sign-magnitude to offset binary); NaN and -inf map to 0, below all.
__device__ __forceinline__ unsigned tq_order_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (v != v || v == -INFINITY) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
}
__device__ __forceinline__ float tq_order_value(unsigned key) {      // the inverse, for key != 0
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// One warp chooses for one row of E <= 32 * SELECT_REGS logits (global or shared memory): a lane keeps its
// logits in registers and a choice is two warp-wide integer reductions.  picks: where the choices go besides
// ids_row (shared memory of the caller), or null.
#define SELECT_REGS 8
template <int NREG>
__device__ __forceinline__ void select_with_registers(const float* row, int E, int k, int renorm, int lane,
                                                      int* __restrict__ ids_row, float* __restrict__ wts_row, int* picks) {
    float v[NREG];
    unsigned key[NREG];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < NREG; ++c) {
        const int e = lane + 32 * c;
        v[c] = e < E ? row[e] : -INFINITY;
        key[c] = e < E ? tq_order_key(v[c]) : 0u;
        mx = fmaxf(mx, v[c]);
    }
    mx = tq_warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < NREG; ++c) if (lane + 32 * c < E) sum += expf(v[c] - mx);
    sum = tq_warp_sum(sum);
    float picked_sum = 0.f, mine = 0.f;             // lane j % 32 keeps the weight of choice j
    for (int j = 0; j < k; ++j) {
        unsigned best = 0;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int c = 0; c < NREG; ++c)
            if (key[c] > best) { best = key[c]; best_e = lane + 32 * c; }      // lower e first within a lane
        const unsigned top = __reduce_max_sync(0xffffffffu, best);
        int pick = __reduce_min_sync(0xffffffffu, (best == top && top != 0u) ? best_e : 0x7fffffff);
        const bool found = pick != 0x7fffffff;
        if (!found) pick = j;                       // nothing left to pick: keep indices valid
        const float p = expf((found ? tq_order_value(top) : -INFINITY) - mx) / sum;
        picked_sum += p;                            // identical in every lane
#pragma unroll
        for (int c = 0; c < NREG; ++c) if (found && lane + 32 * c == pick) key[c] = 0u;
        if (lane == 0) { ids_row[j] = pick; if (picks) picks[j] = pick; }
        if (j < 32) { if (lane == j) mine = p; }
        else if (lane == 0) wts_row[j] = p;         // more than 32 choices: the rest go through memory
    }
    if (lane < k) wts_row[lane] = renorm ? mine / picked_sum : mine;
    if (k > 32 && renorm) {
        __syncwarp();
        for (int j = 32 + lane; j < k; j += 32) wts_row[j] = wts_row[j] / picked_sum;
    }
}

// E <= 32 * SELECT_REGS; the fewer experts, the fewer registers a lane goes through for every choice.
__device__ __forceinline__ void select_in_registers(const float* row, int E, int k, int renorm, int lane,
                                                    int* __restrict__ ids_row, float* __restrict__ wts_row, int* picks) {
    if (E <= 64) select_with_registers<2>(row, E, k, renorm, lane, ids_row, wts_row, picks);
    else if (E <= 128) select_with_registers<4>(row, E, k, renorm, lane, ids_row, wts_row, picks);
    else select_with_registers<SELECT_REGS>(row, E, k, renorm, lane, ids_row, wts_row, picks);
}

// Kernel 2: one warp per token: softmax over the E logits, k largest (ties to the lowest index; NaN never
// wins), weights, shared gate.  Up to 256 experts a lane keeps its logits in registers and a choice is two
// warp-wide integer reductions; beyond that the row is re-read from memory and chosen entries overwritten.
__global__ void router_select_kernel(float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ wts,
                                     float* __restrict__ shared_scale, int T_, int E, int k, int renorm) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T_) return;
    float* s_logit = logits + (size_t)t * (E + 1);      // this warp's row
    if (shared_scale && lane == 0) shared_scale[t] = 1.0f / (1.0f + expf(-s_logit[E]));
    if (E <= 32 * SELECT_REGS) {
        select_in_registers(s_logit, E, k, renorm, lane, ids + (size_t)t * k, wts + (size_t)t * k, nullptr);
        return;
    }
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s_logit[e]);
    mx = tq_warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(s_logit[e] - mx);
    sum = tq_warp_sum(sum);
    float picked_sum = 0.f;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = s_logit[e];
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }   // NaN never wins
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = j;   // every remaining logit is NaN: keep indices valid
        const float p = expf(best - mx) / sum;
        picked_sum += p;                        // identical in every lane
        if (lane == 0) {
            ids[(size_t)t * k + j] = best_e;
            wts[(size_t)t * k + j] = p;
            s_logit[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm) {
        __syncwarp();
        for (int j = lane; j < k; j += 32) wts[(size_t)t * k + j] = wts[(size_t)t * k + j] / picked_sum;
    }
}

// logits: T * (E + 1) floats of scratch.
TQ_EXPORT int tq_router_topk(const void* x, int act_dtype, const void* wr, const void* wsg, int w_dtype,
                             float* logits, int* ids, float* wts, float* shared_scale, int T_, int H, int E, int k,
                             int renorm, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(E >= 1 && E <= ROUTER_MAX_EXPERTS, "router: %d experts exceed %d", E, ROUTER_MAX_EXPERTS);
    TQ_REQUIRE(k >= 1 && k <= E, "router: top-k %d must be in 1..%d", k, E);
    TQ_REQUIRE((wsg == nullptr) == (shared_scale == nullptr), "router: shared gate weight and output must come together");
    TQ_REQUIRE(logits != nullptr, "router: scratch for the logits is required");
    const bool staged = H <= ROUTER_MAX_STAGED_H;
    const size_t smem = staged ? (size_t)H * sizeof(float) : 0;
    const int wbytes = w_dtype == TQ_F32 ? 4 : 2;
    const int vec_ok = ((size_t)H * wbytes) % 16 == 0 && ((uintptr_t)wr % 16) == 0 && (!wsg || ((uintptr_t)wsg % 16) == 0);
    const int rows = E + (wsg ? 1 : 0);
    // few tokens: cut the rows into chunks so that the step still fills the GPU; many tokens: one chunk
    int chunks = T_ >= 256 ? 1 : (512 + T_ - 1) / T_;
    if (chunks > (rows + 3) / 4) chunks = (rows + 3) / 4;
    if (chunks < 1) chunks = 1;
    const int rows_per_cta = (rows + chunks - 1) / chunks;
    chunks = (rows + rows_per_cta - 1) / rows_per_cta;
    const int threads = rows_per_cta >= 32 ? 1024 : (rows_per_cta >= 16 ? 512 : (rows_per_cta >= 8 ? 256 : 128));
    dim3 grid(T_, chunks);
#define ROUTER_LAUNCH(ST)                                                                              \
    TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(w_dtype, TW,                                                \
        (tq_launch(grid, threads, smem, stream)(router_logits_kernel<TA, TW, ST>,                             \
            (const TA*)x, (const TW*)wr, (const TW*)wsg, logits, H, E, rows_per_cta, vec_ok))))
    if (staged) { ROUTER_LAUNCH(true); } else { ROUTER_LAUNCH(false); }
#undef ROUTER_LAUNCH
    TQ_CHECK_LAUNCH("router_logits");
    tq_launch((T_ + 3) / 4, 128, 0, stream)(router_select_kernel, logits, ids, wts, shared_scale, T_, E, k, renorm);
    TQ_CHECK_LAUNCH("router_select");
    return 0;
}

// Selection alone, for logits [T, E + 1] computed elsewhere (the tensor-core GEMM on long prompts).
TQ_EXPORT int tq_router_select(float* logits, int* ids, float* wts, float* shared_scale, int T_, int E, int k,
                               int renorm, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(E >= 1 && E <= ROUTER_MAX_EXPERTS, "router: %d experts exceed %d", E, ROUTER_MAX_EXPERTS);
    TQ_REQUIRE(k >= 1 && k <= E, "router: top-k %d must be in 1..%d", k, E);
    tq_launch((T_ + 3) / 4, 128, 0, stream)(router_select_kernel, logits, ids, wts, shared_scale, T_, E, k, renorm);
    TQ_CHECK_LAUNCH("router_select");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Expert-sorted layout.  Pair p = t*k + j chose expert ids[p].  Rows of the sorted layout:
// expert 0's pairs in pair order, then expert 1's, …  Outputs:
//   sorted_pair[row] = p, row_of_pair[p] = row, expert_offset[e] (E+1 entries),
//   tiles of at most tile_rows rows that never span two experts: tile_expert, tile_row0,
//   tile_count, and n_tiles[0].
// Two kernels over chunks of pairs (512 or more, 256 chunks at most): per-chunk histograms, then every chunk places its pairs.
// ---------------------------------------------------------------------------------------
// Kernel 1: histogram of each chunk of `chunk` pairs.
__global__ void moe_chunk_hist_kernel(const int* __restrict__ ids, int P, int E, int chunk, int* __restrict__ chunk_hist) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ int s_hist[];
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
    __syncthreads();
    const int p0 = blockIdx.x * chunk, p1 = min(P, p0 + chunk);
    for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) atomicAdd(&s_hist[TQ_CHECKED(ids[p], E, TQ_IDX_EXPERT)], 1);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_hist[(size_t)blockIdx.x * E + e] = s_hist[e];
}

// Kernel 2: every block places its chunk.  The row of a pair = rows of the experts before its expert
// + pairs of the same expert in earlier chunks + its rank among the same expert's pairs of this chunk
// (in pair order: the sort is stable).  Block 0 also writes the per-expert tables and the tile list.
__global__ void moe_chunk_place_kernel(const int* __restrict__ ids, int P, int E, int tile_rows, int chunk, int n_chunks,
                                       const int* __restrict__ chunk_hist, int* __restrict__ counts,
                                       int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                                       int* __restrict__ expert_offset, int* __restrict__ tile_expert,
                                       int* __restrict__ tile_row0, int* __restrict__ tile_count,
                                       int* __restrict__ n_tiles) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ int s_mem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* s_total = s_mem;                      // [E]   pairs of each expert
    int* s_run = s_mem + E;                    // [E]   next row of each expert for this block
    int* s_off = s_mem + 2 * E;                // [E+1] first row of each expert
    int* s_toff = s_mem + 3 * E + 1;           // [E+1] first tile of each expert
    int* s_cnt = s_mem + 4 * E + 2;            // [warps][E] pairs of each expert per warp in the current round
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int total = 0, before = 0;
        for (int c = 0; c < n_chunks; ++c) {
            const int h = chunk_hist[(size_t)c * E + e];
            total += h;
            if (c < (int)blockIdx.x) before += h;
        }
        s_total[e] = total;
        s_run[e] = before;
        for (int w = 0; w < warps; ++w) s_cnt[w * E + e] = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            s_off[e] = rows;
            s_toff[e] = tiles;
            rows += s_total[e];
            tiles += (s_total[e] + tile_rows - 1) / tile_rows;
        }
        s_off[E] = rows;
        s_toff[E] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_run[e] += s_off[e];
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e <= E; e += blockDim.x) {
            expert_offset[e] = s_off[e];
            if (e < E) {
                counts[e] = s_total[e];
                // an expert's rows are split evenly over its tiles (136 rows in tiles of 128: 68 + 68, not 128 + 8)
                const int nt = (s_total[e] + tile_rows - 1) / tile_rows;
                for (int i = 0, t = s_toff[e]; i < nt; ++i, ++t) {
                    const int r0 = (int)((long long)s_total[e] * i / nt), r1 = (int)((long long)s_total[e] * (i + 1) / nt);
                    tile_expert[t] = e;
                    tile_row0[t] = s_off[e] + r0;
                    tile_count[t] = r1 - r0;
                }
            }
        }
        if (threadIdx.x == 0) n_tiles[0] = s_toff[E];
    }
    __syncthreads();
    const int p0 = blockIdx.x * chunk, p1 = min(P, p0 + chunk);
    for (int r0 = p0; r0 < p1; r0 += blockDim.x) {
        const int p = r0 + threadIdx.x;
        const int e = p < p1 ? TQ_CHECKED(ids[p], E, TQ_IDX_EXPERT) : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);        // lanes of this warp with the same expert
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const bool leader = rank == 0 && e >= 0;
        if (leader) s_cnt[warp * E + e] = __popc(peers);
        __syncthreads();
        if (e >= 0) {
            int row = s_run[e] + rank;
            for (int w = 0; w < warp; ++w) row += s_cnt[w * E + e];
            sorted_pair[row] = p;
            row_of_pair[p] = row;
        }
        __syncthreads();
        if (leader) {
            atomicAdd(&s_run[e], __popc(peers));
            s_cnt[warp * E + e] = 0;
        }
        __syncthreads();
    }
}

// chunk: pairs per block; chunk_hist: ceil(P / chunk) * E ints of scratch.
TQ_EXPORT int tq_moe_align(const int* ids, int P, int E, int tile_rows, int chunk, int* chunk_hist, int* counts, int* sorted_pair,
                           int* row_of_pair, int* expert_offset, int* tile_expert, int* tile_row0,
                           int* tile_count, int* n_tiles, cudaStream_t stream) {
    TQ_REQUIRE(P >= 0 && E >= 1 && tile_rows >= 1, "moe_align: bad sizes P=%d E=%d tile_rows=%d", P, E, tile_rows);
    TQ_REQUIRE(E <= ROUTER_MAX_EXPERTS, "moe_align: %d experts exceed %d", E, ROUTER_MAX_EXPERTS);
    TQ_REQUIRE(chunk >= 1 && chunk_hist != nullptr, "moe_align: a chunk size and scratch for the chunk histograms are required");
    const int n_chunks = P > 0 ? (P + chunk - 1) / chunk : 1;
    const int threads = E <= 1024 ? 256 : 64;                     // [warps][E] counters must fit shared memory
    tq_launch(n_chunks, threads, (size_t)E * sizeof(int), stream)(moe_chunk_hist_kernel, ids, P, E, chunk, chunk_hist);
    TQ_CHECK_LAUNCH("moe_chunk_hist");
    const size_t smem = (size_t)(4 * E + 2 + (threads / 32) * E) * sizeof(int);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_chunk_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TQ_REQUIRE(e == cudaSuccess, "moe_align: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    }
    tq_launch(n_chunks, threads, smem, stream)(moe_chunk_place_kernel, ids, P, E, tile_rows, chunk, n_chunks, chunk_hist, counts,
                                               sorted_pair, row_of_pair, expert_offset, tile_expert, tile_row0, tile_count,
                                               n_tiles);
    TQ_CHECK_LAUNCH("moe_chunk_place");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Steps with few tokens (decoding): router logits, selection, expert-sorted layout, tile list and the
// expert-sorted copies of the token rows in ONE launch instead of six that each do microseconds of
// work.  Two forms:
//  * up to 8 tokens and 256 experts: eight blocks that are one thread-block cluster.  Block b computes the
//    logits of ITS SHARE OF THE EXPERTS for all tokens (an SM then reads an eighth of the router matrix, which
//    it has asked the L2 for before the kernel ahead of it in the stream was done) and stores them into the
//    shared memory of the block that owns the token; block t chooses for token t; the choices go round through
//    distributed shared memory; every token's block works out the layout for itself and writes the copies of
//    its own row from shared memory; block 0 writes the layout.  Between reading the rows and writing the
//    outputs nothing waits for global memory.
//  * otherwise: one block per token computes that token's logits and choices; the block that finishes last (a
//    counter in global memory) lays out all pairs and copies the rows.  The counter is zero between launches:
//    the last block resets it.  Launches that share a counter must not overlap.
// ---------------------------------------------------------------------------------------
#define SMALL_MAX_PAIRS 512
#define SMALL_MAX_EXPERTS 1023      // the scan over the experts gives thread E the totals: E < blockDim.x
#define SMALL_THREADS 1024
#define SMALL_DYNAMIC_BYTES (27 * 1024)     // what the kernel's own arrays leave of the 48 KiB a block gets without asking
#define SMALL_CLUSTER 8                     // blocks of the cluster form, and the most tokens it takes
#define SMALL_CLUSTER_DYNAMIC_BYTES (160 * 1024)

struct SmallShared {
    int ids[SMALL_MAX_PAIRS], row[SMALL_MAX_PAIRS], mine[SMALL_MAX_PAIRS];
    int count[SMALL_MAX_EXPERTS + 1], off[SMALL_MAX_EXPERTS + 1], toff[SMALL_MAX_EXPERTS + 1];
    int wrows[32], wtiles[32];
};

// Layout of the P pairs whose experts are in S.ids, by all threads of a block of SMALL_THREADS: S.row[row] =
// pair, and for the pairs of token `own` (if >= 0) S.mine[j] = row of its choice j.  writer: this block writes
// the layout to global memory.
__device__ __forceinline__ void small_layout(SmallShared& S, int P, int E, int k, int tile_rows, int own, bool writer,
                                             int* __restrict__ counts, int* __restrict__ sorted_pair,
                                             int* __restrict__ row_of_pair, int* __restrict__ expert_offset,
                                             int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                             int* __restrict__ tile_count, int* __restrict__ n_tiles) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e < E; e += blockDim.x) S.count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&S.count[S.ids[p]], 1);
    __syncthreads();
    {   // offsets of rows and of tiles before expert e: a scan over the experts (E < blockDim.x = 1024)
        const int e = threadIdx.x;
        const int c = e < E ? S.count[e] : 0, tl = (c + tile_rows - 1) / tile_rows;
        int r_incl = c, t_incl = tl;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, r_incl, o), u = __shfl_up_sync(0xffffffffu, t_incl, o);
            if (lane >= o) { r_incl += r; t_incl += u; }
        }
        if (lane == 31) { S.wrows[warp] = r_incl; S.wtiles[warp] = t_incl; }
        __syncthreads();
        if (warp == 0) {
            int r = lane < nwarps ? S.wrows[lane] : 0, u = lane < nwarps ? S.wtiles[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int r2 = __shfl_up_sync(0xffffffffu, r, o), u2 = __shfl_up_sync(0xffffffffu, u, o);
                if (lane >= o) { r += r2; u += u2; }
            }
            S.wrows[lane] = r;                                // inclusive over warps
            S.wtiles[lane] = u;
        }
        __syncthreads();
        const int r_before = (warp > 0 ? S.wrows[warp - 1] : 0) + r_incl - c;
        const int t_before = (warp > 0 ? S.wtiles[warp - 1] : 0) + t_incl - tl;
        if (e <= E) {
            S.off[e] = r_before;
            S.toff[e] = t_before;
            if (writer) {
                expert_offset[e] = r_before;
                if (e < E) counts[e] = c;
                if (e == E) n_tiles[0] = t_before;
            }
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {       // stable: pairs of an expert keep their order
        const int e = S.ids[p];
        int rank = 0;
        for (int q = 0; q < p; ++q) rank += S.ids[q] == e;
        const int row = S.off[e] + rank;
        S.row[row] = p;
        if (p / k == own) S.mine[p % k] = row;
        if (writer) {
            sorted_pair[row] = p;
            row_of_pair[p] = row;
        }
    }
    if (writer)
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const int c = S.count[e], nt = (c + tile_rows - 1) / tile_rows;     // c <= 512: the products fit an int
            for (int i = 0; i < nt; ++i) {                    // an expert's rows split evenly over its tiles
                const int r0 = c * i / nt, r1 = c * (i + 1) / nt;
                tile_expert[S.toff[e] + i] = e;
                tile_row0[S.toff[e] + i] = S.off[e] + r0;
                tile_count[S.toff[e] + i] = r1 - r0;
            }
        }
    __syncthreads();
}

// ---- the cluster form ----
__device__ __forceinline__ unsigned small_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void small_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned small_peer_addr(const void* mine, unsigned rank) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(mine);
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ int small_ld_peer(const int* mine, unsigned rank) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(small_peer_addr(mine, rank)) : "memory");
    return v;
}
__device__ __forceinline__ void small_st_peer(float* mine, unsigned rank, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(small_peer_addr(mine, rank)), "f"(v) : "memory");
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(SMALL_THREADS)
router_cluster_kernel(const TA* __restrict__ x, const TW* __restrict__ wr, const TW* __restrict__ wsg,
                      int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ shared_scale,
                      int T_, int H, int E, int k, int renorm, int vec_dot, int tile_rows,
                      int* __restrict__ counts, int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                      int* __restrict__ expert_offset, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                      int* __restrict__ tile_count, int* __restrict__ n_tiles, TA* __restrict__ x_rows, int vec_x) {
    const unsigned rank = small_cluster_rank();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // a block's shared memory may be written by its peers only once it runs: every block says so here and
    // waits for the others just before its first store
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    // this block's share of the rows of the router matrix (the shared expert's gate row counts as row E)
    const int rows = E + (wsg ? 1 : 0);
    const int per = (rows + SMALL_CLUSTER - 1) / SMALL_CLUSTER;
    const int r0 = min(rows, (int)rank * per), r1 = min(rows, r0 + per);
    {   // the weights do not depend on the kernel before this one: ask the L2 for them while that kernel still
        // runs (between two uses a whole step's weights pass through the L2)
        const long long bytes = (long long)(min(r1, E) - r0) * H * (long long)sizeof(TW);
        const char* base = reinterpret_cast<const char*>(wr + (size_t)r0 * H);
        for (long long off = (long long)threadIdx.x * 128; off < bytes; off += (long long)blockDim.x * 128)
            asm volatile("prefetch.global.L2::evict_last [%0];" ::"l"(base + off));
    }
    uint64_t keep;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep));
    tq_grid_wait();
    tq_grid_launch_dependents();
    extern __shared__ __align__(16) unsigned char s_raw[];
    float* s_logit = reinterpret_cast<float*>(s_raw);                         // [E + 1] the logits of this block's token
    TA* s_x = reinterpret_cast<TA*>(s_raw + (((size_t)(E + 1) * 4 + 15) & ~(size_t)15));   // [T][H] the step's rows
    __shared__ SmallShared S;
    const TA* xs = tq_fresh(x);                                               // loads of x stay behind the wait
    if (vec_x) {
        const int n16 = (int)((size_t)T_ * H * sizeof(TA) / 16);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(s_x)[i] = reinterpret_cast<const uint4*>(xs)[i];
    } else {
        for (int i = threadIdx.x; i < T_ * H; i += blockDim.x) s_x[i] = xs[i];
    }
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");      // all blocks of the cluster run
    // ---- logits of rows [r0, r1) for all tokens, two tokens per pass over a row (the same sums, in the same
    //      order, as router_logits_kernel); each lands in the shared memory of its token's block ----
    const int Hv = vec_dot ? (H / 8) * 8 : 0;
    const int TG = (T_ + 1) / 2;
    for (int item = warp; item < (r1 - r0) * TG; item += nwarps) {
        const int e = r0 + item / TG, t0 = (item % TG) * 2, t1 = min(t0 + 1, T_ - 1);
        const TW* w = e < E ? wr + (size_t)e * H : wsg;
        const TA* xa = s_x + (size_t)t0 * H;
        const TA* xb = s_x + (size_t)t1 * H;
        float s = 0.f, s2 = 0.f;
#pragma unroll 8
        for (int i = lane * 8; i < Hv; i += 256) {
            float f[8], a[8], b[8];
            RowVec<TW>::load_keep(w + i, f, keep);
            RowVec<TA>::load(xa + i, a);
            RowVec<TA>::load(xb + i, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) { s = fmaf(a[j], f[j], s); s2 = fmaf(b[j], f[j], s2); }
        }
        for (int i = Hv + lane; i < H; i += 32) {
            const float f = tq_to_float(w[i]);
            s = fmaf(tq_to_float(xa[i]), f, s);
            s2 = fmaf(tq_to_float(xb[i]), f, s2);
        }
        s = tq_warp_sum(s);
        s2 = tq_warp_sum(s2);
        if (lane == 0) {
            small_st_peer(&s_logit[e], (unsigned)t0, s);
            if (t1 != t0) small_st_peer(&s_logit[e], (unsigned)t1, s2);
        }
    }
    small_cluster_sync();                                     // every token's logits are in its block
    const int t = (int)rank;
    if (t < T_ && warp == 0) {
        if (shared_scale && lane == 0) shared_scale[t] = 1.0f / (1.0f + expf(-s_logit[E]));
        select_in_registers(s_logit, E, k, renorm, lane, ids + (size_t)t * k, wts + (size_t)t * k, S.mine);
    }
    small_cluster_sync();                                     // every token's choices are in its block
    const int P = T_ * k;
    if (t < T_)
        for (int p = threadIdx.x; p < P; p += blockDim.x) S.ids[p] = small_ld_peer(&S.mine[p % k], (unsigned)(p / k));
    small_cluster_sync();                                     // nobody reads a peer's memory after this: blocks may leave
    if (t >= T_) return;
    small_layout(S, P, E, k, tile_rows, t, t == 0, counts, sorted_pair, row_of_pair, expert_offset, tile_expert, tile_row0,
                 tile_count, n_tiles);
    // this token's row, still in shared memory, to each of its k places
    const TA* mine = s_x + (size_t)t * H;
    if (vec_x) {
        const int n16 = (int)((size_t)H * sizeof(TA) / 16);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) {
            const uint4 v = reinterpret_cast<const uint4*>(mine)[i];
            for (int j = 0; j < k; ++j) reinterpret_cast<uint4*>(x_rows + (size_t)S.mine[j] * H)[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x)
            for (int j = 0; j < k; ++j) x_rows[(size_t)S.mine[j] * H + i] = mine[i];
    }
}

// ---- the form for one to four tokens (bfloat16 rows and weights) ----
// One block.  What such a step pays for is trips to memory one after another, not bytes, so: a warp takes rows of
// the router matrix in pairs, its lanes ask for all their 16-byte pieces of the first pair at once and BEFORE the
// kernel waits for the one ahead of it (weights do not depend on it); then the tokens' rows come into shared memory,
// the dots, warp t chooses for token t, and the few pairs are laid out by counting (a pair's row = the pairs with a
// smaller expert, or the same expert and an earlier place): two block barriers, no scan.  Every expert has at most
// one tile (at most four rows, tiles hold at least as many).
#define TINY_MAX_T 4
#define TINY_MAX_PAIRS 64
#define TINY_KI 8
#define TINY_THREADS 512                 // 16 warps: 128 registers a thread, for the two rows a lane holds in flight
__device__ __forceinline__ uint4 tiny_ld16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void tiny_widen(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

template <int T>
__global__ void __launch_bounds__(TINY_THREADS)
router_tiny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr, const __nv_bfloat16* __restrict__ wsg,
                   int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ shared_scale, int H, int E, int k,
                   int renorm, int* __restrict__ counts, int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                   int* __restrict__ expert_offset, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                   int* __restrict__ tile_count, int* __restrict__ n_tiles, __nv_bfloat16* __restrict__ x_rows) {
    extern __shared__ __align__(16) unsigned char s_tiny[];
    __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(s_tiny);                     // [T][H]
    float* s_logit = reinterpret_cast<float*>(s_tiny + (size_t)T * H * 2);             // [T][E + 1]
    __shared__ int s_ids[TINY_MAX_PAIRS], s_row[TINY_MAX_PAIRS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int rows = E + (wsg ? 1 : 0);
    auto row_ptr = [&](int r) { return r < E ? wr + (size_t)r * H : wsg; };
    // the first two rows of this warp, all pieces a lane has in them (up to TINY_KI each), before the wait
    uint4 wa[TINY_KI], wb[TINY_KI];
    auto ask = [&](int r0, int k0) {
        const int r1 = r0 + nwarps;
#pragma unroll
        for (int it = 0; it < TINY_KI; ++it) {
            const int kk = k0 + lane * 8 + it * 256;
            wa[it] = (r0 < rows && kk < H) ? tiny_ld16(row_ptr(r0) + kk) : make_uint4(0u, 0u, 0u, 0u);
            wb[it] = (r1 < rows && kk < H) ? tiny_ld16(row_ptr(r1) + kk) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    ask(warp, 0);
    tq_grid_wait();
    tq_grid_launch_dependents();
    const __nv_bfloat16* xs = tq_fresh(x);                 // loads of x stay behind the wait
    for (int i = threadIdx.x * 8; i < T * H; i += blockDim.x * 8)
        *reinterpret_cast<uint4*>(s_x + i) = *reinterpret_cast<const uint4*>(xs + i);
    __syncthreads();
    // ---- logits (fp32 sums of the bf16 products, a lane's pieces in order, then the lanes by shuffles) ----
    for (int r0 = warp; r0 < rows; r0 += 2 * nwarps) {
        const int r1 = r0 + nwarps;
        float sa[T], sb[T];
#pragma unroll
        for (int t = 0; t < T; ++t) { sa[t] = 0.f; sb[t] = 0.f; }
        for (int k0 = 0; k0 < H; k0 += TINY_KI * 256) {
            if (r0 != warp || k0 != 0) ask(r0, k0);          // the first pieces were asked for before the wait
#pragma unroll
            for (int it = 0; it < TINY_KI; ++it) {
                const int kk = k0 + lane * 8 + it * 256;
                if (kk < H) {
                    float fa[8], fb[8];
                    tiny_widen(wa[it], fa);
                    tiny_widen(wb[it], fb);
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        float xf[8];
                        tiny_widen(*reinterpret_cast<const uint4*>(s_x + (size_t)t * H + kk), xf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) { sa[t] = fmaf(xf[i], fa[i], sa[t]); sb[t] = fmaf(xf[i], fb[i], sb[t]); }
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const float va = tq_warp_sum(sa[t]), vb = tq_warp_sum(sb[t]);
            if (lane == 0) {
                s_logit[t * (E + 1) + r0] = va;
                if (r1 < rows) s_logit[t * (E + 1) + r1] = vb;
            }
        }
    }
    __syncthreads();
    // ---- warp t chooses for token t ----
    if (warp < T) {
        const float* row = s_logit + warp * (E + 1);
        if (shared_scale && lane == 0) shared_scale[warp] = 1.0f / (1.0f + expf(-row[E]));
        select_in_registers(row, E, k, renorm, lane, ids + (size_t)warp * k, wts + (size_t)warp * k, s_ids + warp * k);
    }
    __syncthreads();
    // ---- layout by counting ----
    const int P = T * k;
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        int below = 0, own = 0, tiles_below = 0;
        for (int q = 0; q < P; ++q) {
            const int id = s_ids[q];
            below += id < e;
            own += id == e;
            if (id < e) {                                   // count an expert once: at its first pair
                bool firstq = true;
                for (int q2 = 0; q2 < q; ++q2) firstq = firstq && s_ids[q2] != id;
                tiles_below += firstq;
            }
        }
        expert_offset[e] = below;
        if (e < E) {
            counts[e] = own;
            if (own > 0) { tile_expert[tiles_below] = e; tile_row0[tiles_below] = below; tile_count[tiles_below] = own; }
        } else {
            n_tiles[0] = tiles_below;
        }
    }
    if (threadIdx.x < P) {
        const int p = threadIdx.x, id = s_ids[p];
        int row = 0;
        for (int q = 0; q < P; ++q) row += (s_ids[q] < id) || (s_ids[q] == id && q < p);
        s_row[p] = row;
        sorted_pair[row] = p;
        row_of_pair[p] = row;
    }
    __syncthreads();
    // ---- the tokens' rows, still in shared memory, to their pairs' places ----
    const int n16 = H / 8;
    for (int i = threadIdx.x; i < P * n16; i += blockDim.x) {
        const int p = i / n16, c = i - p * n16;
        reinterpret_cast<uint4*>(x_rows + (size_t)s_row[p] * H)[c] = reinterpret_cast<const uint4*>(s_x + (size_t)(p / k) * H)[c];
    }
}

// ---- the counter form ----
template <typename TA, typename TW>
__global__ void __launch_bounds__(SMALL_THREADS)
router_small_kernel(const TA* __restrict__ x, const TW* __restrict__ wr, const TW* __restrict__ wsg,
                    int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ shared_scale,
                    int T_, int H, int E, int k, int renorm, int vec_w, int tile_rows,
                    int* __restrict__ counts, int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                    int* __restrict__ expert_offset, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                    int* __restrict__ tile_count, int* __restrict__ n_tiles, TA* __restrict__ x_rows, int vec_x,
                    int* __restrict__ counter) {
    tq_grid_wait();
    tq_grid_launch_dependents();
    extern __shared__ float s_dyn[];
    float* s_x = s_dyn;               // [H] the token's row
    float* s_logit = s_dyn + H;       // [E + 1] router logits, then the shared expert's gate logit
    __shared__ SmallShared S;
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const TA* xr = x + (size_t)t * H;
    // ---- this token's logits (the same sums, in the same order, as router_logits_kernel) ----
    for (int i = threadIdx.x; i < H; i += blockDim.x) s_x[i] = tq_to_float(xr[i]);
    __syncthreads();
    const int rows = E + (wsg ? 1 : 0);
    const int Hv = vec_w ? (H / 8) * 8 : 0;
    // two rows per warp at a time and the loop unrolled: all of a step's loads are in flight together (the
    // work is a few hundred KB; what counts is the number of dependent trips to memory)
    for (int e = warp; e < rows; e += 2 * nwarps) {
        const int e2 = e + nwarps < rows ? e + nwarps : e;
        const TW* w = e < E ? wr + (size_t)e * H : wsg;
        const TW* w2 = e2 < E ? wr + (size_t)e2 * H : wsg;
        float s = 0.f, s2 = 0.f;
#pragma unroll 8
        for (int i = lane * 8; i < Hv; i += 256) {
            float f[8], f2[8];
            RowVec<TW>::load(w + i, f);
            RowVec<TW>::load(w2 + i, f2);
#pragma unroll
            for (int j = 0; j < 8; ++j) { s = fmaf(s_x[i + j], f[j], s); s2 = fmaf(s_x[i + j], f2[j], s2); }
        }
        for (int i = Hv + lane; i < H; i += 32) {
            s = fmaf(s_x[i], tq_to_float(w[i]), s);
            s2 = fmaf(s_x[i], tq_to_float(w2[i]), s2);
        }
        s = tq_warp_sum(s);
        s2 = tq_warp_sum(s2);
        if (lane == 0) { s_logit[e] = s; s_logit[e2] = s2; }      // e2 == e: the same value twice
    }
    __syncthreads();
    // ---- selection: warp 0 (the same choices and weights as router_select_kernel) ----
    if (warp == 0) {
        if (shared_scale && lane == 0) shared_scale[t] = 1.0f / (1.0f + expf(-s_logit[E]));
        if (E <= 32 * SELECT_REGS) {
            select_in_registers(s_logit, E, k, renorm, lane, ids + (size_t)t * k, wts + (size_t)t * k, nullptr);
        } else {
            float mx = -INFINITY;
            for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s_logit[e]);
            mx = tq_warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < E; e += 32) sum += expf(s_logit[e] - mx);
            sum = tq_warp_sum(sum);
            float* s_val = s_x;                               // the row is no longer needed: its place holds the k picked logits
            for (int j = 0; j < k; ++j) {
                // largest remaining logit, ties to the lowest index; NaN and -inf (already picked) never win
                unsigned best = 0;
                int best_e = 0x7fffffff;
                for (int e = lane; e < E; e += 32) {
                    const unsigned key = tq_order_key(s_logit[e]);
                    if (key > best) { best = key; best_e = e; }   // lower e first within a lane
                }
                const unsigned top = __reduce_max_sync(0xffffffffu, best);
                int pick = __reduce_min_sync(0xffffffffu, (best == top && top != 0u) ? best_e : 0x7fffffff);
                if (pick == 0x7fffffff) pick = j;             // nothing left to pick: keep indices valid
                if (lane == 0) {
                    ids[(size_t)t * k + j] = pick;
                    s_val[j] = top != 0u ? s_logit[pick] : -INFINITY;
                    s_logit[pick] = -INFINITY;
                }
                __syncwarp();
            }
            // weights: lanes take the exponentials, every lane adds them up in the order of the choices
            for (int j = lane; j < k; j += 32) s_val[j] = expf(s_val[j] - mx) / sum;
            __syncwarp();
            float picked_sum = 0.f;
            if (renorm) for (int j = 0; j < k; ++j) picked_sum += s_val[j];
            for (int j = lane; j < k; j += 32) wts[(size_t)t * k + j] = renorm ? s_val[j] / picked_sum : s_val[j];
        }
        __threadfence();                                      // this token's choices are visible before the count
        __syncwarp();
        if (lane == 0) s_last = atomicAdd(counter, 1) == T_ - 1;
    }
    __syncthreads();
    if (!s_last) return;
    // ---- the last block: layout of all pairs, tile list, expert-sorted copies of the rows ----
    __threadfence();
    const int P = T_ * k;
    for (int p = threadIdx.x; p < P; p += blockDim.x) S.ids[p] = __ldcg(ids + p);
    __syncthreads();
    small_layout(S, P, E, k, tile_rows, -1, true, counts, sorted_pair, row_of_pair, expert_offset, tile_expert, tile_row0,
                 tile_count, n_tiles);
    for (int row = warp; row < P; row += nwarps) {            // expert-sorted copies of the token rows
        const TA* src = x + (size_t)(S.row[row] / k) * H;
        TA* dst = x_rows + (size_t)row * H;
        if (vec_x) {
            const int n16 = (int)((size_t)H * sizeof(TA) / 16);
            const uint4* s4 = reinterpret_cast<const uint4*>(src);
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            for (int i0 = lane; i0 < n16; i0 += 256) {          // eight 16-byte loads in flight per lane, then the stores
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) if (i0 + 32 * j < n16) v[j] = s4[i0 + 32 * j];
#pragma unroll
                for (int j = 0; j < 8; ++j) if (i0 + 32 * j < n16) d4[i0 + 32 * j] = v[j];
            }
        } else {
            for (int i = lane; i < H; i += 32) dst[i] = src[i];
        }
    }
    if (threadIdx.x == 0) *counter = 0;                       // ready for the next launch
}

template <typename TA, typename TW, typename... Args>
static cudaError_t launch_router_cluster(size_t smem, cudaStream_t stream, Args... args) {
    auto kern = router_cluster_kernel<TA, TW>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMALL_CLUSTER_DYNAMIC_BYTES);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    tq_launch(SMALL_CLUSTER, SMALL_THREADS, smem, stream, SMALL_CLUSTER)(kern, args...);
    return cudaSuccess;
}

// Router, expert-sorted layout and gathered rows for a step of few tokens, in one launch.
// Needs T*k <= 512 pairs, E <= 1023 experts and (H + E + 1) floats of shared memory within 27 KiB;
// counter: one int in device memory, zero before the first launch (the kernel leaves it zero).
TQ_EXPORT int tq_router_small(const void* x, int act_dtype, const void* wr, const void* wsg, int w_dtype,
                              int* ids, float* wts, float* shared_scale, int tile_rows, int* counts, int* sorted_pair,
                              int* row_of_pair, int* expert_offset, int* tile_expert, int* tile_row0, int* tile_count,
                              int* n_tiles, void* x_rows, int* counter, int T_, int H, int E, int k, int renorm,
                              cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ * k <= SMALL_MAX_PAIRS && E <= SMALL_MAX_EXPERTS,
               "router_small: %d pairs / %d experts exceed %d / %d", T_ * k, E, SMALL_MAX_PAIRS, SMALL_MAX_EXPERTS);
    TQ_REQUIRE(E >= 1 && k >= 1 && k <= E && tile_rows >= 1, "router_small: bad sizes E=%d k=%d tile_rows=%d", E, k, tile_rows);
    TQ_REQUIRE((wsg == nullptr) == (shared_scale == nullptr), "router: shared gate weight and output must come together");
    TQ_REQUIRE(counter != nullptr, "router_small: a counter is required");
    const size_t smem = (size_t)(H + E + 1) * sizeof(float);
    TQ_REQUIRE(smem <= SMALL_DYNAMIC_BYTES, "router_small: a row of %d values and %d logits do not fit %d bytes of shared memory",
               H, E, SMALL_DYNAMIC_BYTES);
    const int wbytes = w_dtype == TQ_F32 ? 4 : 2;
    const int vec_w = ((size_t)H * wbytes) % 16 == 0 && ((uintptr_t)wr % 16) == 0 && (!wsg || ((uintptr_t)wsg % 16) == 0);
    const int abytes = act_dtype == TQ_F32 ? 4 : 2;
    const int vec_x = ((size_t)H * abytes) % 16 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)x_rows % 16) == 0;
    // one token in bfloat16: the single-block form (TQ_ROUTER_NO_TINY=1: the others after all).  The kernel takes up
    // to four tokens, but inside a decode step it only wins with one (measured on B200, tokens/s of the step with
    // this form / with the cluster: 538 / 518 at batch 1, 942 / 940 at batch 2, 1,380 / 1,455 at batch 4).
    {
        const char* tiny_env = getenv("TQ_ROUTER_NO_TINY");
        const bool no_tiny = tiny_env && tiny_env[0] && tiny_env[0] != '0';
        const size_t smem_tiny = (size_t)T_ * H * 2 + (size_t)T_ * (E + 1) * 4;
        if (!no_tiny && (T_ == 1 || (tiny_env && tiny_env[0] == '0' && T_ <= TINY_MAX_T)) && T_ * k <= TINY_MAX_PAIRS && T_ <= tile_rows && act_dtype == TQ_BF16 && w_dtype == TQ_BF16 &&
            H % 8 == 0 && vec_w && vec_x && E <= 32 * SELECT_REGS && smem_tiny <= 40 * 1024) {
#define TINY_CASE(TT) case TT: tq_launch(1, TINY_THREADS, smem_tiny, stream)(router_tiny_kernel<TT>, (const __nv_bfloat16*)x, \
            (const __nv_bfloat16*)wr, (const __nv_bfloat16*)wsg, ids, wts, shared_scale, H, E, k, renorm, counts, sorted_pair,  \
            row_of_pair, expert_offset, tile_expert, tile_row0, tile_count, n_tiles, (__nv_bfloat16*)x_rows); break;
            switch (T_) { TINY_CASE(1) TINY_CASE(2) TINY_CASE(3) TINY_CASE(4) }
#undef TINY_CASE
            TQ_CHECK_LAUNCH("router_tiny");
            return 0;
        }
    }
    // the cluster form (TQ_ROUTER_NO_CLUSTER=1: the counter form after all)
    const size_t smem_cluster = (((size_t)(E + 1) * 4 + 15) & ~(size_t)15) + (size_t)T_ * H * abytes;
    const char* no_cluster = getenv("TQ_ROUTER_NO_CLUSTER");
    const bool cluster = T_ <= SMALL_CLUSTER && E <= 32 * SELECT_REGS && smem_cluster <= SMALL_CLUSTER_DYNAMIC_BYTES &&
                         (vec_x || !vec_w) &&       // the order of a sum follows the weights' loads; the rows must allow the same
                         !(no_cluster && no_cluster[0] && no_cluster[0] != '0');
    if (cluster) {
        const int vec_dot = vec_w;                            // 16-byte loads of the weights and of the rows in shared memory
        cudaError_t cfg = cudaSuccess;
        TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(w_dtype, TW,
            (cfg = launch_router_cluster<TA, TW>(smem_cluster, stream, (const TA*)x, (const TW*)wr, (const TW*)wsg,
                ids, wts, shared_scale, T_, H, E, k, renorm, vec_dot, tile_rows, counts, sorted_pair, row_of_pair, expert_offset,
                tile_expert, tile_row0, tile_count, n_tiles, (TA*)x_rows, vec_x))));
        TQ_REQUIRE(cfg == cudaSuccess, "router_small: %zu bytes of shared memory refused: %s", smem_cluster, cudaGetErrorString(cfg));
    } else {
        TQ_DISPATCH(act_dtype, TA, TQ_DISPATCH(w_dtype, TW,
            (tq_launch(T_, SMALL_THREADS, smem, stream)(router_small_kernel<TA, TW>, (const TA*)x, (const TW*)wr, (const TW*)wsg,
                ids, wts, shared_scale, T_, H, E, k, renorm, vec_w, tile_rows, counts, sorted_pair, row_of_pair, expert_offset,
                tile_expert, tile_row0, tile_count, n_tiles, (TA*)x_rows, vec_x, counter))));
    }
    TQ_CHECK_LAUNCH("router_small");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Exact grouped GEMM on CUDA cores.  A [R, K]; W [G, Nw, K] with Nw = N (plain) or 2N (SwiGLU:
// gate rows [0, N), up rows [N, 2N)); C [R, N].  Rows come in tiles (tile_expert/row0/count);
// with tile_expert == null there is one group and tile b covers rows [b*64, b*64+64).
// Every output element is one sequential fp32 sum over K, so it does not depend on the tile the
// row falls in.
// ---------------------------------------------------------------------------------------
#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <typename TA, typename TW, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ C,
                    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    const int* __restrict__ tile_count, const int* __restrict__ n_tiles,
                    int R, int N, int K) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[SWIGLU ? 2 : 1][GG_BK][GG_BN + 4];
    int expert = 0, row0, rows;
    if (tile_expert) {
        if ((int)blockIdx.y >= n_tiles[0]) return;
        expert = tile_expert[blockIdx.y];
        row0 = tile_row0[blockIdx.y];
        rows = tile_count[blockIdx.y];
    } else {
        row0 = blockIdx.y * GG_BM;
        if (row0 >= R) return;
        rows = min(GG_BM, R - row0);
    }
    const int n0 = blockIdx.x * GG_BN;
    const int Nw = SWIGLU ? 2 * N : N;
    const TW* Wg = W + (size_t)expert * Nw * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // 16 x 16 threads, 4 x 4 outputs each
    float acc[SWIGLU ? 2 : 1][4][4];
#pragma unroll
    for (int s = 0; s < (SWIGLU ? 2 : 1); ++s)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = 0.f;

    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row 0..63, k 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int kk = k0 + lk + u;
            float a = 0.f;
            if (lr < rows && kk < K) a = tq_to_float(A[(size_t)(row0 + lr) * K + kk]);
            As[lk + u][lr] = a;
            const int n = n0 + lr;
            float w0 = 0.f;
            if (n < N && kk < K) w0 = tq_to_float(Wg[(size_t)n * K + kk]);
            Ws[0][lk + u][lr] = w0;
            if (SWIGLU) {
                float w1 = 0.f;
                if (n < N && kk < K) w1 = tq_to_float(Wg[(size_t)(N + n) * K + kk]);
                Ws[SWIGLU ? 1 : 0][lk + u][lr] = w1;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int s = 0; s < (SWIGLU ? 2 : 1); ++s) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Ws[s][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[s][i][j] = fmaf(a[i], b[j], acc[s][i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v;
            if (SWIGLU) {
                const float g = acc[0][i][j], u = acc[SWIGLU ? 1 : 0][i][j];
                v = g / (1.0f + expf(-g)) * u;
            } else {
                v = acc[0][i][j];
            }
            C[(size_t)(row0 + r) * N + n] = tq_from_float<TO>(v);
        }
    }
}

// ---------------------------------------------------------------------------------------
// The same product for tiles of a few rows (decode steps), as a stream of the weights: a block stages
// GV_ROWS rows of its tile in shared memory (in pieces of GV_KC values of K) and each warp computes one output
// column (with SwiGLU: from a gate and an up row) for all of them, a lane taking every 32nd group of four values of K, the lanes' sums added by shuffles.
// The tiled kernel above reads a 64-row tile's worth of weights for however few rows the tile holds and keeps few
// loads in flight; this one keeps several 16-byte pieces of a weight row in flight per lane (measured on B200 in
// float32 at 60 experts of 1408 x 2048: a decode step of 8 tokens 39.0 -> 14.5 ms, of one token 18.8 -> 3.0 ms with
// two rows per pass and eight pieces in flight; eight rows and four pieces: 21 and 5.6 ms; four output columns per warp
// were 10 % faster than one at 8 tokens and took six times as long to compile).  fp32 multiply-adds in a fixed order that
// depends on K alone: a row's result does not depend on the tile it falls in or on the rest of the batch.
// ---------------------------------------------------------------------------------------
#define GV_ROWS 2
#define GV_WARPS 8
#define GV_KC 2048                 // values of K per piece: 4 rows x 2048 floats = 32 KiB of shared memory
#define GV_FLY 8                   // 16-byte pieces of a weight row a lane has in flight

// four weights at p as floats (16-byte or 8-byte load; the caller made sure of the alignment)
template <typename T> __device__ __forceinline__ float4 gv_load4(const T* p);
template <> __device__ __forceinline__ float4 gv_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 gv_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename TA, typename TW, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(GV_WARPS * 32)
grouped_gemv_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ C,
                    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                    const int* __restrict__ tile_count, const int* __restrict__ n_tiles,
                    int R, int N, int K, int tile_rows, int vec) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ __align__(16) float s_rows[];          // [GV_ROWS][GV_KC]
    int expert = 0, row0, rows;
    if (tile_expert) {
        if ((int)blockIdx.y >= n_tiles[0]) return;
        expert = tile_expert[blockIdx.y];
        row0 = tile_row0[blockIdx.y];
        rows = tile_count[blockIdx.y];
    } else {
        row0 = blockIdx.y * tile_rows;
        if (row0 >= R) return;
        rows = min(tile_rows, R - row0);
    }
    constexpr int S = SWIGLU ? 2 : 1;
    constexpr int COLS = 1;                                            // output columns of a warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int Nw = SWIGLU ? 2 * N : N;
    const TW* Wg = W + (size_t)expert * Nw * K;
    const int n_first = (blockIdx.x * GV_WARPS + warp) * COLS;         // this warp's columns
    for (int rb = 0; rb < rows; rb += GV_ROWS) {                       // usually one trip: a tile of a decode step is short
        const int nr = min(GV_ROWS, rows - rb);
        float acc[COLS][S][GV_ROWS];
#pragma unroll
        for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r) acc[c][s][r] = 0.f;
        for (int k0 = 0; k0 < K; k0 += GV_KC) {
            const int kc = min(GV_KC, K - k0);
            __syncthreads();                                           // the piece before this one has been used
            // all GV_ROWS rows of the piece, rows the tile does not have and values past the piece's end as zeros: the
            // sums below then need no conditions
            const int kc4 = (kc + 3) & ~3;
            for (int i = threadIdx.x; i < GV_ROWS * kc4; i += blockDim.x) {
                const int r = i / kc4, kk = i - r * kc4;
                s_rows[r * GV_KC + kk] = (r < nr && kk < kc) ? tq_to_float(A[(size_t)(row0 + rb + r) * K + k0 + kk]) : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
                const int n = n_first + c;
                if (n < N) {                                           // uniform across the warp
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        const TW* wrow = Wg + (size_t)(s * N + n) * K + k0;
                        // a lane takes every 32nd group of four values; GV_FLY groups are asked for before the first is used
                        for (int kb = lane * 4; kb < kc; kb += 128 * GV_FLY) {
                            float4 w4[GV_FLY];
#pragma unroll
                            for (int f = 0; f < GV_FLY; ++f) {
                                const int kk = kb + 128 * f;
                                if (vec) {
                                    w4[f] = kk < kc ? gv_load4<TW>(wrow + kk) : make_float4(0.f, 0.f, 0.f, 0.f);
                                } else {
                                    w4[f].x = kk < kc ? tq_to_float(wrow[kk]) : 0.f;
                                    w4[f].y = kk + 1 < kc ? tq_to_float(wrow[kk + 1]) : 0.f;
                                    w4[f].z = kk + 2 < kc ? tq_to_float(wrow[kk + 2]) : 0.f;
                                    w4[f].w = kk + 3 < kc ? tq_to_float(wrow[kk + 3]) : 0.f;
                                }
                            }
#pragma unroll
                            for (int f = 0; f < GV_FLY; ++f) {
                                const int kk = kb + 128 * f < kc ? kb + 128 * f : 0;   // a group past the end has zero weights: any staged values do
#pragma unroll
                                for (int r = 0; r < GV_ROWS; ++r) {
                                    const float4 a = *reinterpret_cast<const float4*>(s_rows + r * GV_KC + kk);
                                    float t = acc[c][s][r];
                                    t = fmaf(a.x, w4[f].x, t);
                                    t = fmaf(a.y, w4[f].y, t);
                                    t = fmaf(a.z, w4[f].z, t);
                                    t = fmaf(a.w, w4[f].w, t);
                                    acc[c][s][r] = t;
                                }
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
            const int n = n_first + c;
            if (n < N) {
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r) {
                    if (r < nr) {
                        float v = tq_warp_sum(acc[c][0][r]);
                        if (SWIGLU) {
                            const float u = tq_warp_sum(acc[c][S - 1][r]);
                            v = v / (1.0f + expf(-v)) * u;
                        }
                        if (lane == 0) C[(size_t)(row0 + rb + r) * N + n] = tq_from_float<TO>(v);
                    }
                }
            }
        }
    }
}

// tile_rows: the rows of a tile when there is no tile list (one group); few_rows != 0 selects this kernel in
// tq_grouped_gemm.
template <typename TA, typename TW, typename TO, bool SWIGLU>
int launch_grouped_gemv(const void* A, const void* W, void* C, const int* te, const int* tr, const int* tc, const int* nt,
                        int by, int R, int N, int K, int tile_rows, cudaStream_t stream) {
    auto kern = grouped_gemv_kernel<TA, TW, TO, SWIGLU>;
    const int smem = GV_ROWS * GV_KC * (int)sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) TQ_FAIL(-1, "grouped_gemm: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    constexpr int cols = GV_WARPS;
    dim3 grid((N + cols - 1) / cols, by);
    // 16-byte (8-byte) loads of four weights: rows of K values that start on such a boundary
    const int vec = K % 4 == 0 && ((uintptr_t)W % (4 * sizeof(TW))) == 0;
    tq_launch(grid, GV_WARPS * 32, smem, stream)(kern, (const TA*)A, (const TW*)W, (TO*)C, te, tr, tc, nt, R, N, K, tile_rows, vec);
    return 0;
}

TQ_EXPORT int tq_grouped_gemm(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                              const int* tile_expert, const int* tile_row0, const int* tile_count,
                              const int* n_tiles, int max_tiles, int R, int N, int K, int swiglu, int few_rows,
                              cudaStream_t stream) {
    if (R == 0 || (tile_expert && max_tiles == 0)) return 0;
    TQ_REQUIRE(R > 0 && N > 0 && K > 0, "grouped_gemm: bad sizes R=%d N=%d K=%d", R, N, K);
    const int by = tile_expert ? max_tiles : (R + GG_BM - 1) / GG_BM;
    TQ_REQUIRE(by <= 65535, "grouped_gemm: %d row tiles exceed the grid limit", by);
    // tiles of a few rows each (a decode step): the weight-stream form, for the type combinations the parts use
    // (all float32; bfloat16 in and out; bfloat16 in, float32 out); others take the tiled kernel
    const bool gv_types = (a_dtype == TQ_F32 && w_dtype == TQ_F32 && c_dtype == TQ_F32) ||
                          (a_dtype == TQ_BF16 && w_dtype == TQ_BF16);
    if (few_rows && gv_types) {
        int rc = 0;
#define GV_LAUNCH(TA, TW, TO)                                                                                     \
        rc = swiglu ? launch_grouped_gemv<TA, TW, TO, true>(A, W, C, tile_expert, tile_row0, tile_count, n_tiles, by, R, N, K, GG_BM, stream) \
                    : launch_grouped_gemv<TA, TW, TO, false>(A, W, C, tile_expert, tile_row0, tile_count, n_tiles, by, R, N, K, GG_BM, stream)
        if (a_dtype == TQ_F32) GV_LAUNCH(float, float, float);
        else if (c_dtype == TQ_F32) GV_LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
        else GV_LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
#undef GV_LAUNCH
        if (rc) return rc;
        TQ_CHECK_LAUNCH("grouped_gemv");
        return 0;
    }
    dim3 grid((N + GG_BN - 1) / GG_BN, by);
#define GG_LAUNCH(SW)                                                                                   \
    TQ_DISPATCH(a_dtype, TA, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(c_dtype, TO,                          \
        (tq_launch(grid, 256, 0, stream)(grouped_gemm_kernel<TA, TW, TO, SW>,                                  \
            (const TA*)A, (const TW*)W, (TO*)C, tile_expert, tile_row0, tile_count, n_tiles, R, N, K)))))
    if (swiglu) { GG_LAUNCH(true); } else { GG_LAUNCH(false); }
#undef GG_LAUNCH
    TQ_CHECK_LAUNCH("grouped_gemm");
    return 0;
}

// ---------------------------------------------------------------------------------------
// y[t] = sum_j wts[t,j] * Y[row_of_pair[t*k+j]] + shared_scale[t] * sum_s Ys[s][t]   (fp32; Ys holds `parts`
// slices [T][H]: the shared expert's output, or its partial sums over shares of K, added in slice order)
// ---------------------------------------------------------------------------------------
__global__ void moe_combine_kernel(const float* __restrict__ Y, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ wts, const float* __restrict__ Ys,
                                   const float* __restrict__ shared_scale, float* __restrict__ y, int H, int k, int R,
                                   int parts) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    if ((H & 3) == 0) {          // four columns per thread, 16-byte accesses (rows of fp32 are 16-byte aligned)
        const float sc = Ys ? (shared_scale ? shared_scale[t] : 1.0f) : 0.f;
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < H; i += gridDim.y * blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int j = 0; j < k; ++j) {                   // unrolled: the chosen experts' rows load side by side
                const float wj = wts[(size_t)t * k + j];
                const float4 a = *reinterpret_cast<const float4*>(Y + (size_t)TQ_CHECKED(row_of_pair[(size_t)t * k + j], R, TQ_IDX_ROW) * H + i);
                v.x += wj * a.x; v.y += wj * a.y; v.z += wj * a.z; v.w += wj * a.w;
            }
            if (Ys) {
                float4 a = *reinterpret_cast<const float4*>(Ys + (size_t)t * H + i);
                for (int sp = 1; sp < parts; ++sp) {
                    const float4 b = *reinterpret_cast<const float4*>(Ys + ((size_t)sp * gridDim.x + t) * H + i);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                }
                v.x += sc * a.x; v.y += sc * a.y; v.z += sc * a.z; v.w += sc * a.w;
            }
            *reinterpret_cast<float4*>(y + (size_t)t * H + i) = v;
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float v = 0.f;
        for (int j = 0; j < k; ++j)
            v += wts[(size_t)t * k + j] * Y[(size_t)TQ_CHECKED(row_of_pair[(size_t)t * k + j], R, TQ_IDX_ROW) * H + i];
        if (Ys) {
            float a = Ys[(size_t)t * H + i];
            for (int sp = 1; sp < parts; ++sp) a += Ys[((size_t)sp * gridDim.x + t) * H + i];
            v += (shared_scale ? shared_scale[t] : 1.0f) * a;
        }
        y[(size_t)t * H + i] = v;
    }
}

// R: rows of Y (what row_of_pair is checked against in a debug build).  parts: slices of Ys, [parts][T][H].
TQ_EXPORT int tq_moe_combine(const float* Y, const int* row_of_pair, const float* wts, const float* Ys,
                             const float* shared_scale, float* y, int T_, int H, int k, int R, int parts,
                             cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(H > 0 && k >= 0 && parts >= 1, "moe_combine: bad sizes H=%d k=%d parts=%d", H, k, parts);
    // few tokens: narrow blocks, several per row, so that the step still fills the GPU
    const int threads = T_ >= 512 ? 256 : 64;
    int cols = T_ >= 512 ? 1 : (H + threads * 4 - 1) / (threads * 4);
    if (cols > 64) cols = 64;
    tq_launch(dim3(T_, cols), threads, 0, stream)(moe_combine_kernel, Y, row_of_pair, wts, Ys, shared_scale, y, H, k, R, parts);
    TQ_CHECK_LAUNCH("moe_combine");
    return 0;
}
