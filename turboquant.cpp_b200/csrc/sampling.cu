// Sampling from rows of fp32 logits: argmax, and temperature with a nucleus (top-p).
//
// The reference samples on the CPU (src/engine/tq_generate.c): argmax takes the first maximum
// (:30-40); top-p (:81-156) keeps logits >= max - 16*T, forms p = exp((l - max)/T), sorts by p
// descending, cuts where the cumulative sum reaches top_p, draws r = u * cumulative and walks the
// sorted list until the running sum reaches r.  The kernel below picks the same token without a
// sort: "the first element in sorted order whose prefix sum reaches a target" is found by a
// bisection on the value p (32 block-wide sums) and, among equal values, by index order.
// One block per row; the uniform u of each row is an input, so a draw depends on the caller's
// (seed, sequence, step) only.
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

#define SAMPLE_THREADS 1024

// ---------------------------------------------------------------------------------------
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
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
        if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;   // all NaN: token 0, as the reference
    }
}

TQ_EXPORT int tq_argmax_rows(const float* logits, int R, int V, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && V > 0, "argmax_rows: bad sizes R=%d V=%d", R, V);
    tq_launch(R, V >= 4096 ? 1024 : 256, 0, stream)(argmax_rows_kernel, logits, V, out);
    TQ_CHECK_LAUNCH("argmax_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// Sum over the row of p[i] for which pred holds; every thread gets the result.
// ---------------------------------------------------------------------------------------
struct PrefixPick { float value; float above; int ties; };

// Finds the value v* = the largest v with sum_{p >= v} p >= target, the mass strictly above it and
// the number of elements equal to it.  p holds V non-negative floats (0 = not a candidate).
__device__ PrefixPick find_crossing(const float* __restrict__ p, int V, float target, float* scratch) {
    unsigned lo = 1u, hi = 0x3f800000u;        // bit patterns of the smallest positive float .. 1.0f
    // invariant: A(lo) >= target (or lo is the floor), A(hi + 1) < target
    while (lo < hi) {
        const unsigned mid = lo + (hi - lo + 1) / 2;
        const float v = __uint_as_float(mid);
        float s = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) { const float x = p[i]; if (x >= v) s += x; }
        s = tq_block_sum(s, scratch);
        if (s >= target) lo = mid; else hi = mid - 1;
    }
    PrefixPick r;
    r.value = __uint_as_float(lo);
    float above = 0.f, ties = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = p[i];
        if (x > r.value) above += x; else if (x == r.value) ties += 1.f;
    }
    r.above = tq_block_sum(above, scratch);
    r.ties = (int)tq_block_sum(ties, scratch);
    return r;
}

__global__ void sample_rows_kernel(const float* __restrict__ logits, int V, float temperature, float top_p,
                                   const float* __restrict__ uniforms, float* __restrict__ work,
                                   int* __restrict__ out) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    __shared__ int s_warp[SAMPLE_THREADS / 32];
    __shared__ int s_base, s_found;
    const float* row = logits + (size_t)blockIdx.x * V;
    float* p = work + (size_t)blockIdx.x * V;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = tq_block_max(mx, scratch);
    const float thr = mx - 16.0f * temperature, inv_t = 1.0f / temperature;
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = row[i];
        const float e = l >= thr ? expf((l - mx) * inv_t) : 0.f;
        p[i] = e;
        z += e;
    }
    z = tq_block_sum(z, scratch);          // also orders the writes of p before the reads below
    // the nucleus: the cut element is the first whose prefix sum reaches top_p * z
    float mass = z;
    if (top_p < 1.0f) {
        const PrefixPick cut = find_crossing(p, V, top_p * z, scratch);
        int n = (int)ceilf((top_p * z - cut.above) / cut.value);
        n = max(1, min(n, cut.ties));
        mass = cut.above + (float)n * cut.value;
    }
    const float r = uniforms[blockIdx.x] * mass;
    PrefixPick pick = find_crossing(p, V, r, scratch);
    int n = (int)ceilf((r - pick.above) / pick.value);
    n = max(1, min(n, pick.ties));
    // the n-th element (in index order) whose value equals pick.value
    if (threadIdx.x == 0) { s_base = 0; s_found = -1; }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i0 = 0; i0 < V && s_found < 0; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        const bool tie = i < V && p[i] == pick.value;
        const unsigned ballot = __ballot_sync(0xffffffffu, tie);
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        int before = s_base;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        const int rank = before + __popc(ballot & ((1u << lane) - 1u)) + 1;
        if (tie && rank == n) s_found = i;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_warp[w];
            s_base += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = s_found >= 0 ? s_found : 0;
}

// work: R*V floats of scratch.
TQ_EXPORT int tq_sample_rows(const float* logits, int R, int V, float temperature, float top_p,
                             const float* uniforms, float* work, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && V > 0, "sample_rows: bad sizes R=%d V=%d", R, V);
    TQ_REQUIRE(temperature > 0.f && top_p > 0.f, "sample_rows: temperature %g and top_p %g must be positive "
               "(use argmax_rows otherwise)", (double)temperature, (double)top_p);
    tq_launch(R, SAMPLE_THREADS, 0, stream)(sample_rows_kernel, logits, V, temperature, top_p, uniforms, work, out);
    TQ_CHECK_LAUNCH("sample_rows");
    return 0;
}
