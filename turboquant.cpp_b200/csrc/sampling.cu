// Sampling from rows of fp32 logits: argmax, and temperature with a nucleus (top-p).
//
// The reference samples on the CPU (src/engine/tq_generate.c): argmax takes the first maximum
// (:30-40); top-p (:81-156) keeps logits >= max - 16*T, forms p = exp((l - max)/T), sorts by p
// descending, cuts where the cumulative sum reaches top_p, draws r = u * cumulative and walks the
// sorted list until the running sum reaches r.  The kernel below picks the same token without a
// sort: "the first element in sorted order whose prefix sum reaches a target" is found by a
// search on the value p (sixteen bins of bit patterns per pass, each thread adding into a column of its
// own, seven passes over [2^-24, 1]) and, among equal values, by index order.  A row is shared by a cluster of up to eight CTAs,
// each with its slice of p in shared memory; partial sums cross the cluster through distributed shared
// memory and are added in rank order, so every CTA sees the same totals and takes the same branches.
// All sums have a fixed order: a draw is reproducible, and the sum over a superset is never smaller.
// The uniform u of each row is an input, so a draw depends on the caller's (seed, sequence, step) only.
//
// Before it samples, the reference lowers the logits of the tokens it saw last (:586-600, the first token
// :386-399): for each of the last `window` tokens of the request, once per occurrence, a positive logit is
// divided by the penalty and any other multiplied by it.  tq_rep_penalty does the same in place.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define SAMPLE_THREADS 512

// ---------------------------------------------------------------------------------------
// Cluster plumbing
// ---------------------------------------------------------------------------------------
#define SAMPLE_BINS 16                      // the search cuts its range into this many parts per pass
#define SAMPLE_MAX_CLUSTER 8
#define SAMPLE_SLICE_MIN 4096               // a CTA's share of a row is at least this long
#define SAMPLE_SMEM_FLOATS 45056            // longer slices keep p in global scratch instead of shared memory

__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer(const float* mine, unsigned rank) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(mine);
    unsigned r;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------
// grid = rows x cluster size; a CTA scans `slice` columns of its row, rank 0 picks among the CTAs' results.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, int slice, int* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ float s_best;           // read by rank 0 through the cluster's shared memory
    __shared__ float s_best_i;         // the index's bits, carried as a float
    const unsigned rank = cluster_rank(), csize = cluster_size();
    const int row_id = blockIdx.x / csize;
    const int first = (int)rank * slice, last = min(V, first + slice);
    const float* row = logits + (size_t)row_id * V;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
#pragma unroll 4
    for (int i = first + threadIdx.x; i < last; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_v[warp] = best; s_i[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nwarps ? s_v[lane] : -INFINITY;
        best_i = lane < nwarps ? s_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { s_best = best; s_best_i = __int_as_float(best_i); }
    }
    cluster_sync();
    if (rank == 0 && threadIdx.x == 0) {
        for (unsigned q = 1; q < csize; ++q) {          // slices follow one another: an equal value further on loses
            const float ov = ld_peer(&s_best, q);
            const int oi = __float_as_int(ld_peer(&s_best_i, q));
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        out[row_id] = best_i == 0x7fffffff ? 0 : best_i;   // all NaN: token 0, as the reference
    }
    cluster_sync();                    // nobody leaves while rank 0 may still read its result
}

static int row_cluster(int V) {
    int cluster = (V + SAMPLE_SLICE_MIN - 1) / SAMPLE_SLICE_MIN;
    cluster = cluster > SAMPLE_MAX_CLUSTER ? SAMPLE_MAX_CLUSTER : cluster;
    while (cluster & (cluster - 1)) cluster &= cluster - 1;          // 1, 2, 4 or 8
    return cluster;
}

TQ_EXPORT int tq_argmax_rows(const float* logits, int R, int V, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && V > 0, "argmax_rows: bad sizes R=%d V=%d", R, V);
    const int cluster = row_cluster(V), slice = (V + cluster - 1) / cluster;
    tq_launch(R * cluster, slice >= 4096 ? 1024 : 256, 0, stream, cluster)(argmax_rows_kernel, logits, V, slice, out);
    TQ_CHECK_LAUNCH("argmax_rows");
    return 0;
}

static_assert(SAMPLE_BINS == SAMPLE_THREADS / 32, "one warp folds each bin");
struct Exchange {
    float bins[SAMPLE_BINS][SAMPLE_THREADS];    // the search's partial sums: a column per thread
    float warp_part[SAMPLE_THREADS / 32][2];
    float mine[2][SAMPLE_BINS];     // this CTA's partials, two generations: peers read one while the next is written
    float total[SAMPLE_BINS];
};

// Reduces K per-thread values over the whole cluster (MAX: maximum, else sum); every thread of every CTA
// gets the same K results in x.total.  `gen` flips with every call.  After the call, x.mine[gen_used][j] of
// rank r still holds that rank's partial until the call after the next.
template <int K, bool MAX>          // K <= 2
__device__ __forceinline__ void cluster_reduce(float (&v)[K], Exchange& x, int& gen) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int j = 0; j < K; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], o);
            v[j] = MAX ? fmaxf(v[j], other) : v[j] + other;
        }
        if (lane == 0) x.warp_part[warp][j] = v[j];
    }
    __syncthreads();
    if (warp < K) {                 // warp j folds value j of all warps, again as a tree
        float t = lane < nwarps ? x.warp_part[lane][warp] : (MAX ? -INFINITY : 0.f);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, t, o);
            t = MAX ? fmaxf(t, other) : t + other;
        }
        if (lane == 0) x.mine[gen][warp] = t;
    }
    cluster_sync();
    if (threadIdx.x < K) {
        const unsigned n = cluster_size();
        float part[SAMPLE_MAX_CLUSTER];
#pragma unroll
        for (unsigned r = 0; r < SAMPLE_MAX_CLUSTER; ++r)           // all loads in flight, then added in rank order
            part[r] = r < n ? ld_peer(&x.mine[gen][threadIdx.x], r) : (MAX ? -INFINITY : 0.f);
        float t = part[0];
#pragma unroll
        for (unsigned r = 1; r < SAMPLE_MAX_CLUSTER; ++r) t = MAX ? fmaxf(t, part[r]) : t + part[r];
        x.total[threadIdx.x] = t;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < K; ++j) v[j] = x.total[j];
    __syncthreads();                // x.total and x.warp_part may be written again
    gen ^= 1;
}

struct PrefixPick { float value; float above; int ties; int gen; };

// Finds the value v* = the largest v with sum_{p >= v} p >= target, the mass strictly above it and
// the number of elements equal to it.  p holds this CTA's n slice elements, non-negative (0 = not a candidate).
// pick.gen names the generation of x.mine that holds every rank's (above, ties) partials.
__device__ PrefixPick find_crossing(const float* p, int n, float target, Exchange& x, int& gen) {
    unsigned lo = 0x33800000u, hi = 0x3f800000u;   // bit patterns of 2^-24 (below every candidate's exp(-16)) .. 1.0f
    // invariant: A(lo) >= target (or lo is the floor), A(hi + 1) < target
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    while (lo < hi) {
        // bins of 2^k bit patterns from lo on, the last one open-ended; 16 * 2^k > hi - lo
        const int k = 32 - __clz((hi - lo) >> 4);
#pragma unroll
        for (int b = 0; b < SAMPLE_BINS; ++b) x.bins[b][threadIdx.x] = 0.f;     // each thread its own column
        for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) {
            const float e = p[i];
            const unsigned bits = __float_as_uint(e);
            if (bits >= lo) x.bins[min((bits - lo) >> k, (unsigned)(SAMPLE_BINS - 1))][threadIdx.x] += e;
        }
        __syncthreads();
        {   // warp b folds bin b: the columns in a fixed order, then a tree
            float t = 0.f;
#pragma unroll
            for (int c = 0; c < SAMPLE_THREADS / 32; ++c) t += x.bins[warp][lane + 32 * c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) x.mine[gen][warp] = t;
        }
        cluster_sync();
        if (threadIdx.x < SAMPLE_BINS) {
            const unsigned nr = cluster_size();
            float part[SAMPLE_MAX_CLUSTER];
#pragma unroll
            for (unsigned r = 0; r < SAMPLE_MAX_CLUSTER; ++r)       // all loads in flight, then added in rank order
                part[r] = r < nr ? ld_peer(&x.mine[gen][threadIdx.x], r) : 0.f;
            float t = part[0];
#pragma unroll
            for (unsigned r = 1; r < SAMPLE_MAX_CLUSTER; ++r) t += part[r];
            x.total[threadIdx.x] = t;
        }
        __syncthreads();
        float above = 0.f;                     // sum of the bins from j up = the sum of all p >= lo + j * 2^k
        unsigned best = 0;
#pragma unroll
        for (int j = SAMPLE_BINS - 1; j >= 1; --j) {
            above += x.total[j];
            if (best == 0 && above >= target && lo + ((unsigned)j << k) <= hi) best = (unsigned)j;   // (a target of 0
                                               // is reached by the empty sum beyond hi too)
        }
        __syncthreads();                       // x.total and the bins may be written again
        gen ^= 1;
        hi = min(hi, lo + ((best + 1u) << k) - 1u);
        lo += best << k;
    }
    PrefixPick r;
    r.value = __uint_as_float(lo);
    for (int attempt = 0; attempt < 2; ++attempt) {
        float at[2] = {0.f, 0.f};
        for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) {
            const float e = p[i];
            if (e > r.value) at[0] += e; else if (e == r.value) at[1] += 1.f;
        }
        r.gen = gen;
        cluster_reduce<2, false>(at, x, gen);
        r.above = at[0];
        r.ties = (int)at[1];
        if (r.ties > 0 || attempt == 1) break;
        // No element has this value: the passes' sums, each added in its own order, disagreed in the last bit
        // about a target that lies within rounding of a step of A, most often of its last one (u close to 1:
        // the walk through the sorted list ends at the smallest candidate).  The element meant is the smallest
        // one from here up.
        float neg[1] = {-INFINITY};
        for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) {
            const float e = p[i];
            if (e >= r.value) neg[0] = fmaxf(neg[0], -e);
        }
        cluster_reduce<1, true>(neg, x, gen);
        if (neg[0] == -INFINITY) break;        // no candidate at all
        r.value = -neg[0];
    }
    return r;
}

// grid = rows x cluster size; row_len = V; slice = elements per CTA.
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_rows_kernel(const float* __restrict__ logits, int V, int slice, float temperature, float top_p,
                   const float* __restrict__ uniforms, float* __restrict__ work, int p_in_global,
                   int* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    extern __shared__ float p_shared[];
    __shared__ Exchange x;
    __shared__ int s_warp[SAMPLE_THREADS / 32];
    __shared__ int s_base, s_found;
    const unsigned rank = cluster_rank(), csize = cluster_size();
    const int row_id = blockIdx.x / csize;
    const int first = (int)rank * slice;
    const int n = max(0, min(slice, V - first));
    const float* row = logits + (size_t)row_id * V + first;
    float* p = p_in_global ? work + (size_t)row_id * V + first : p_shared;
    int gen = 0;

    // every thread keeps to its own elements of p (i = thread, thread + 512, ...) in all passes
    float mx[1] = {-INFINITY};
#pragma unroll 8
    for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) {
        const float l = row[i];
        p[i] = l;
        mx[0] = fmaxf(mx[0], l);
    }
    cluster_reduce<1, true>(mx, x, gen);
    const float thr = mx[0] - 16.0f * temperature, inv_t = 1.0f / temperature;
    float z[1] = {0.f};
    for (int i = threadIdx.x; i < n; i += SAMPLE_THREADS) {
        const float l = p[i];
        const float e = l >= thr ? expf((l - mx[0]) * inv_t) : 0.f;
        p[i] = e;
        z[0] += e;
    }
    cluster_reduce<1, false>(z, x, gen);
    // the nucleus: the cut element is the first whose prefix sum reaches top_p * z
    float mass = z[0];
    if (top_p < 1.0f) {
        const PrefixPick cut = find_crossing(p, n, top_p * z[0], x, gen);
        int m = (int)ceilf((top_p * z[0] - cut.above) / cut.value);
        m = max(1, min(m, cut.ties));
        mass = cut.above + (float)m * cut.value;
    }
    const float r = uniforms[row_id] * mass;
    const PrefixPick pick = find_crossing(p, n, r, x, gen);
    int nth = (int)ceilf((r - pick.above) / pick.value);
    nth = max(1, min(nth, pick.ties));
    // the nth element (in index order) whose value equals pick.value: slices follow one another in rank
    // order, so it lies in the CTA whose ties begin before nth and end at or after it
    int before = 0;
    for (unsigned q = 0; q < rank; ++q) before += (int)ld_peer(&x.mine[pick.gen][1], q);
    const int here = (int)x.mine[pick.gen][1];
    if (threadIdx.x == 0) { s_base = before; s_found = -1; }
    __syncthreads();
    if (nth > before && nth <= before + here) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int i0 = 0; i0 < n && s_found < 0; i0 += blockDim.x) {
            const int i = i0 + threadIdx.x;
            const bool tie = i < n && p[i] == pick.value;
            const unsigned ballot = __ballot_sync(0xffffffffu, tie);
            if (lane == 0) s_warp[warp] = __popc(ballot);
            __syncthreads();
            int seen = s_base;
            for (int w = 0; w < warp; ++w) seen += s_warp[w];
            const int idx = seen + __popc(ballot & ((1u << lane) - 1u)) + 1;
            if (tie && idx == nth) s_found = first + i;
            __syncthreads();
            if (threadIdx.x == 0) {
                int tot = 0;
                for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_warp[w];
                s_base += tot;
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) out[row_id] = s_found >= 0 ? s_found : 0;
    } else if (pick.ties == 0 && rank == 0 && threadIdx.x == 0) {
        out[row_id] = 0;               // no candidate at all (every logit NaN): token 0, as argmax does
    }
    cluster_sync();                    // nobody leaves while a peer may still read its partials
}

// work: R*V floats of scratch (used when a CTA's slice of a row does not fit shared memory, or on request).
TQ_EXPORT int tq_sample_rows(const float* logits, int R, int V, float temperature, float top_p,
                             const float* uniforms, float* work, int p_in_global, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && V > 0, "sample_rows: bad sizes R=%d V=%d", R, V);
    TQ_REQUIRE(temperature > 0.f && top_p > 0.f, "sample_rows: temperature %g and top_p %g must be positive "
               "(use argmax_rows otherwise)", (double)temperature, (double)top_p);
    const int cluster = row_cluster(V), slice = (V + cluster - 1) / cluster;
    if (slice > SAMPLE_SMEM_FLOATS) p_in_global = 1;
    const size_t smem = p_in_global ? 0 : (size_t)slice * sizeof(float);
    static size_t smem_set = 0;
    if (smem > smem_set) {
        cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TQ_REQUIRE(e == cudaSuccess, "sample_rows: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        smem_set = smem;
    }
    tq_launch(R * cluster, SAMPLE_THREADS, smem, stream, cluster)(sample_rows_kernel, logits, V, slice, temperature,
                                                                  top_p, uniforms, work, p_in_global, out);
    TQ_CHECK_LAUNCH("sample_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Repetition penalty.  recent [R, W]: the last tokens of each row's request, -1 where it has fewer.
// One thread per row walks its W entries in order, so a token that occurs twice is lowered twice,
// as in the reference's loop, and no two threads touch the same logit.
// ---------------------------------------------------------------------------------------
__global__ void rep_penalty_kernel(float* __restrict__ logits, int R, int V, const int* __restrict__ recent, int W,
                                   float penalty) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    float* row = logits + (size_t)r * V;
    for (int j = 0; j < W; ++j) {
        const int tok = recent[(size_t)r * W + j];
        if (tok < 0 || tok >= V) continue;
        const float x = row[tok];
        row[tok] = x > 0.f ? x / penalty : x * penalty;
    }
}

TQ_EXPORT int tq_rep_penalty(float* logits, int R, int V, const int* recent, int W, float penalty, cudaStream_t stream) {
    if (R == 0 || W == 0) return 0;
    TQ_REQUIRE(R > 0 && V > 0 && W > 0, "rep_penalty: bad sizes R=%d V=%d W=%d", R, V, W);
    TQ_REQUIRE(penalty > 0.f, "rep_penalty: the penalty %g must be positive", (double)penalty);
    tq_launch((R + 63) / 64, 64, 0, stream)(rep_penalty_kernel, logits, R, V, recent, W, penalty);
    TQ_CHECK_LAUNCH("rep_penalty");
    return 0;
}
