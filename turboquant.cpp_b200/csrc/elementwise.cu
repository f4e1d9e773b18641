// Row-wise kernels: embedding rows, RMSNorm (with the residual sum and a row gather fused in),
// SiLU(gate)*up, row gather.  All statistics and the residual sum are computed in fp32.
//
// Formulas as the reference computes them on the CPU:
//   embedding  x = table[token]                       src/engine/tq_transformer.c:2298-2329
//   rmsnorm    ss = sum(x^2)/n + eps; y = x*(1/sqrt(ss))*w   src/engine/tq_ops.c:1373-1410
//   silu       x/(1+exp(-x))                          src/engine/tq_ops.c:1454-1478
#include "common.cuh"

TQ_DEFINE_LAST_ERROR

// ---------------------------------------------------------------------------------------
// x[t, :] = table[tokens[t], :]  (fp32 residual stream out)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                  float* __restrict__ x, int H, int V) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const TW* row = table + (size_t)TQ_CHECKED(tokens[t], V, TQ_IDX_TOKEN) * H;
    float* out = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = tq_to_float(row[i]);
}

TQ_EXPORT int tq_embed_rows(const int* tokens, const void* table, int table_dtype, float* x,
                            int T, int H, int V, cudaStream_t stream) {
    if (T == 0) return 0;
    TQ_REQUIRE(T > 0 && H > 0, "embed_rows: bad sizes T=%d H=%d", T, H);
    const int threads = H >= 1024 ? 256 : 128;
    TQ_DISPATCH(table_dtype, TW,
        tq_launch(T, threads, 0, stream)(embed_rows_kernel<TW>, tokens, (const TW*)table, x, H, V));
    TQ_CHECK_LAUNCH("embed_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------
// RMSNorm over rows of the fp32 residual stream.
//   y given:    the norm is taken of x + y (the residual sum, in fp32)
//   rows given: the norm of row rows[r] is written to out[r] and x is not changed;
//               otherwise row r goes to out[r] and, with y, the sum is written back into x
// ---------------------------------------------------------------------------------------
template <typename TY, typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                               const TW* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (yr) v += tq_to_float(yr[i]);
        if (write_back) xr[i] = v;
        ss += v * v;
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (yr && !write_back) v += tq_to_float(yr[i]);
        o[i] = tq_from_float<TO>(v * rs * tq_to_float(w[i]));
    }
}

// The same with 16-byte accesses: a thread keeps up to 8 groups of 4 elements of its row in registers
// between the two passes (H a multiple of 4, at most 32 * blockDim elements).
template <typename T> __device__ __forceinline__ float4 tq_load4(const T* p);
template <> __device__ __forceinline__ float4 tq_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 tq_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void tq_store4(T* p, float4 v);
template <> __device__ __forceinline__ void tq_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void tq_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

#define RMS_VEC_GROUPS 8
template <typename TY, typename TW, typename TO>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                                   const TW* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    const int nvec = H >> 2;
    float4 v[RMS_VEC_GROUPS], g[RMS_VEC_GROUPS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RMS_VEC_GROUPS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec) {
            g[c] = tq_load4<TW>(w + 4 * i);                 // fetched now, so that it arrives during the reduction
            float4 a = tq_load4<float>(xr + 4 * i);
            if (yr) { const float4 b = tq_load4<TY>(yr + 4 * i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
            if (write_back) tq_store4<float>(xr + 4 * i, a);
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            v[c] = a;
        }
    }
    ss = tq_block_sum(ss, scratch);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < RMS_VEC_GROUPS; ++c) {
        const int i = threadIdx.x + c * blockDim.x;
        if (i < nvec)
            tq_store4<TO>(o + 4 * i, make_float4(v[c].x * rs * g[c].x, v[c].y * rs * g[c].y, v[c].z * rs * g[c].z,
                                                 v[c].w * rs * g[c].w));
    }
}

// Many rows (prompts): a warp per row, the row in registers (up to 16 groups of 4 elements per lane: H <= 2048, a
// multiple of 4), the sums by shuffles: no block-wide barrier, and a lane's loads are all in flight together.
#define RMS_WARP_GROUPS 16
#define RMS_WARP_ROWS 8          // warps (rows) per block
template <typename TY, typename TW, typename TO>
__global__ void __launch_bounds__(32 * RMS_WARP_ROWS)
rmsnorm_warp_kernel(float* __restrict__ x, const TY* __restrict__ y, const int* __restrict__ rows,
                    const TW* __restrict__ w, TO* __restrict__ out, int R, int H, float eps) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * RMS_WARP_ROWS + (threadIdx.x >> 5);
    if (r >= R) return;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src * H;
    const TY* yr = y ? y + src * H : nullptr;
    const bool write_back = y && !rows;
    const int nvec = H >> 2;
    float4 v[RMS_WARP_GROUPS];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) v[c] = tq_load4<float>(xr + 4 * i);
    }
    if (yr) {
#pragma unroll
        for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
            const int i = lane + 32 * c;
            if (i < nvec) { const float4 b = tq_load4<TY>(yr + 4 * i); v[c].x += b.x; v[c].y += b.y; v[c].z += b.z; v[c].w += b.w; }
        }
    }
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) {
            if (write_back) tq_store4<float>(xr + 4 * i, v[c]);
            ss += v[c].x * v[c].x + v[c].y * v[c].y + v[c].z * v[c].z + v[c].w * v[c].w;
        }
    }
    ss = tq_warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
#pragma unroll
    for (int c = 0; c < RMS_WARP_GROUPS; ++c) {
        const int i = lane + 32 * c;
        if (i < nvec) {
            const float4 g = tq_load4<TW>(w + 4 * i);
            tq_store4<TO>(o + 4 * i, make_float4(v[c].x * rs * g.x, v[c].y * rs * g.y, v[c].z * rs * g.z, v[c].w * rs * g.w));
        }
    }
}

TQ_EXPORT int tq_rmsnorm(float* x, const void* y, int y_dtype, const int* rows, const void* w, int w_dtype,
                         void* out, int out_dtype, int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0, "rmsnorm: bad sizes R=%d H=%d", R, H);
    if (H % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)w % 16) == 0 &&
        ((uintptr_t)out % 16) == 0) {
        if (R >= 512 && H / 4 <= 32 * RMS_WARP_GROUPS) {
            TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
                (tq_launch((R + RMS_WARP_ROWS - 1) / RMS_WARP_ROWS, 32 * RMS_WARP_ROWS, 0, stream)(
                    rmsnorm_warp_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w, (TO*)out, R, H, eps)))));
            TQ_CHECK_LAUNCH("rmsnorm");
            return 0;
        }
        int vthreads = ((H / 4 + 31) / 32) * 32;
        if (vthreads > 256 && H / 4 <= 256 * RMS_VEC_GROUPS) vthreads = ((H / 4 + 255) / 256 <= 4) ? 256 : 512;
        if (vthreads > 1024) vthreads = 1024;
        if (H / 4 <= vthreads * RMS_VEC_GROUPS) {
            TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
                (tq_launch(R, vthreads, 0, stream)(rmsnorm_vec_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w,
                                                                            (TO*)out, H, eps)))));
            TQ_CHECK_LAUNCH("rmsnorm");
            return 0;
        }
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    TQ_DISPATCH(y_dtype, TY, TQ_DISPATCH(w_dtype, TW, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(R, threads, 0, stream)(rmsnorm_kernel<TY, TW, TO>, x, (const TY*)y, rows, (const TW*)w,
                                                              (TO*)out, H, eps)))));
    TQ_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------------------
// x[r] += y[r]  (fp32 residual stream; used where no norm follows the sum)
// ---------------------------------------------------------------------------------------
template <typename TY>
__global__ void residual_add_kernel(float* __restrict__ x, const TY* __restrict__ y, size_t n) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] += tq_to_float(y[i]);
}

TQ_EXPORT int tq_residual_add(float* x, const void* y, int y_dtype, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TQ_DISPATCH(y_dtype, TY,
        tq_launch((int)blocks, threads, 0, stream)(residual_add_kernel<TY>, x, (const TY*)y, (size_t)n));
    TQ_CHECK_LAUNCH("residual_add");
    return 0;
}

// ---------------------------------------------------------------------------------------
// x[t, i] += bias[i], in place, summed in fp32 (for a projection whose bias no fused kernel adds)
// ---------------------------------------------------------------------------------------
template <typename TX, typename TB>
__global__ void add_bias_kernel(TX* __restrict__ x, const TB* __restrict__ bias, int N) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    TX* row = x + (size_t)blockIdx.x * N;
    for (int i = threadIdx.x; i < N; i += blockDim.x)
        row[i] = tq_from_float<TX>(tq_to_float(row[i]) + tq_to_float(bias[i]));
}

TQ_EXPORT int tq_add_bias(void* x, int x_dtype, const void* bias, int bias_dtype, int T_, int N, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && N > 0, "add_bias: bad sizes T=%d N=%d", T_, N);
    TQ_DISPATCH(x_dtype, TX, TQ_DISPATCH(bias_dtype, TB,
        (tq_launch(T_, 256, 0, stream)(add_bias_kernel<TX, TB>, (TX*)x, (const TB*)bias, N))));
    TQ_CHECK_LAUNCH("add_bias");
    return 0;
}

// ---------------------------------------------------------------------------------------
// h[t, i] = silu(gu[t, i]) * gu[t, I + i]   (gate rows first, then up rows)
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ h, int I) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int t = blockIdx.x;
    const TI* g = gu + (size_t)t * 2 * I;
    TO* o = h + (size_t)t * I;
    for (int i = threadIdx.x; i < I; i += blockDim.x) {
        const float a = tq_to_float(g[i]), b = tq_to_float(g[I + i]);
        o[i] = tq_from_float<TO>(a / (1.0f + expf(-a)) * b);
    }
}

TQ_EXPORT int tq_silu_mul(const void* gu, int in_dtype, void* h, int out_dtype, int T_, int I, cudaStream_t stream) {
    if (T_ == 0) return 0;
    TQ_REQUIRE(T_ > 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T_, I);
    TQ_DISPATCH(in_dtype, TI, TQ_DISPATCH(out_dtype, TO,
        (tq_launch(T_, 256, 0, stream)(silu_mul_kernel<TI, TO>, (const TI*)gu, (TO*)h, I))));
    TQ_CHECK_LAUNCH("silu_mul");
    return 0;
}

// ---------------------------------------------------------------------------------------
// out[r, :] = in[idx[r] / divisor, :]   (expert-sorted copies of token rows: divisor = top-k)
// ---------------------------------------------------------------------------------------
// A warp copies a row (16-byte accesses when rows allow it); a block takes several rows.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ in, const int* __restrict__ idx, int divisor,
                                   T* __restrict__ out, int R, int H, int vec, int S) {
    tq_grid_wait();                    // everything below may read what the previous kernel wrote
    tq_grid_launch_dependents();       // the next kernel's CTAs may move in as SMs free up
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < R; r += gridDim.x * warps) {
        const T* src = in + (size_t)TQ_CHECKED(idx[r] / divisor, S, TQ_IDX_ROW) * H;
        T* dst = out + (size_t)r * H;
        if (vec) {          // rows are a multiple of 16 bytes and 16-byte aligned
            const int n16 = (int)((size_t)H * sizeof(T) / 16);
            const uint4* s4 = reinterpret_cast<const uint4*>(src);
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            for (int i0 = lane; i0 < n16; i0 += 256) {      // eight 16-byte loads in flight per lane, then the stores
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
}

// S: rows of `in` (what the indices are checked against in a debug build).
TQ_EXPORT int tq_gather_rows(const void* in, const int* idx, int divisor, void* out, int dtype, int R, int H, int S,
                             cudaStream_t stream) {
    if (R == 0) return 0;
    TQ_REQUIRE(R > 0 && H > 0 && divisor > 0, "gather_rows: bad sizes R=%d H=%d divisor=%d", R, H, divisor);
    const int esize = dtype == TQ_F32 ? 4 : 2;
    const int vec = ((size_t)H * esize) % 16 == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0;
    int blocks = (R + 7) / 8;                     // eight warps, a row each, per block
    if (blocks > 148 * 8) blocks = 148 * 8;
    TQ_DISPATCH(dtype, T,
        tq_launch(blocks, 256, 0, stream)(gather_rows_kernel<T>, (const T*)in, idx, divisor, (T*)out, R, H, vec, S));
    TQ_CHECK_LAUNCH("gather_rows");
    return 0;
}
