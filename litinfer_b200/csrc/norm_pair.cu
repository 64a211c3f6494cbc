// Norms around a sublayer ("sandwich" arrangement) as one pass over the residual stream, and two small
// helpers of the same family.
//
//   li_norm_add_norm: per token row
//       x += post(y)          post: a norm of the sublayer's output y with its own weight (or none: x += y; or no y at all)
//       out = next(x)         next: the norm that feeds the following sublayer (optional; without one, out may still be
//                             asked for and is x in the run dtype: a sublayer that reads the stream itself)
//     where a norm is  (v - mean) / sqrt(var + eps) * w  (centered 1: layer norm without bias, var the mean of the squared
//     deviations),  v / sqrt(mean(v^2) + eps) * w  (centered 0: RMS norm)  or just  v * w  (centered 2: a factor per channel).  Rows may be gathered (rows[r]) when
//     there is no y: the model's last norm on the wanted rows only.
//   li_add_row: x[t] += table[row] for every token (a vector per pass of a looped span of layers).
//   li_rmsnorm_cols: RMS norm of n columns of a run-dtype matrix, written to (up to) two places of another matrix.
//
// All sums, means and the residual stream are float; y and out are in the run dtype.  One block per row.  The variance
// is the mean of squared deviations, not a difference of large sums: rows of up to 8,192 elements are held in registers
// for that (read once), longer ones are read again from cache.
#include "common.cuh"

namespace {

// what `centered` says of a norm: 0 an RMS norm, 1 a layer norm without bias, 2 no statistic at all: the row times the weight
// (a learned factor per channel on a sublayer's output)
constexpr int kScaleOnly = 2;

template <typename T>
__device__ __forceinline__ float row_stat_norm(const T* __restrict__ v, int H, int centered, float eps, float* scratch, float* mean_out) {
    float mean = 0.0f;
    if (centered) {
        float s = 0.0f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) s += to_float(v[i]);
        mean = block_sum(s, scratch) / (float)H;
    }
    float q = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = to_float(v[i]) - mean;
        q = fmaf(d, d, q);
    }
    q = block_sum(q, scratch);
    *mean_out = mean;
    return 1.0f / sqrtf(q / (float)H + eps);
}

template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ w_post, int post_centered,
                                     float eps_post, const float* __restrict__ w_next, int next_centered, float eps_next,
                                     T* __restrict__ out, const int* __restrict__ rows, int n_src, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src = r;
    if (rows) {
        src = rows[r];
        if (src < 0 || src >= n_src) src = 0;
    }
    float* xr = x + (size_t)src * H;
    if (y) {
        const T* yr = y + (size_t)r * H;
        if (w_post && post_centered == kScaleOnly) {
            for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] += to_float(yr[i]) * w_post[i];
        } else if (w_post) {
            float mean;
            const float rinv = row_stat_norm(yr, H, post_centered, eps_post, scratch, &mean);
            for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] += (to_float(yr[i]) - mean) * rinv * w_post[i];
        } else {
            for (int i = threadIdx.x; i < H; i += blockDim.x) xr[i] += to_float(yr[i]);
        }
        __syncthreads();                                  // the row's new values are read by other threads below
    }
    if (w_next && next_centered == kScaleOnly) {
        T* o = out + (size_t)r * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<T>(xr[i] * w_next[i]);
    } else if (w_next) {
        float mean;
        const float rinv = row_stat_norm(xr, H, next_centered, eps_next, scratch, &mean);
        T* o = out + (size_t)r * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<T>((xr[i] - mean) * rinv * w_next[i]);
    } else if (out) {
        // no following norm but an output: the row as it is, in the run dtype (a sublayer that reads the stream itself)
        T* o = out + (size_t)r * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<T>(xr[i]);
    }
}

// The same with the row in registers, so that the row of y and the row of x are read once and every moment is taken from
// registers.  kVec (H a multiple of 8): a thread holds 8 neighbouring elements and moves them with 16-byte loads and
// stores; else thread i holds elements i, i + blockDim, ... (up to kRegs of them).  H <= kRegs * blockDim.
constexpr int kRegs = 8;

template <bool kVec>
__device__ __forceinline__ int reg_index(int k) { return kVec ? (int)threadIdx.x * kRegs + k : (int)threadIdx.x + k * (int)blockDim.x; }

template <bool kVec>
__device__ __forceinline__ void load_row(float (&v)[kRegs], const float* __restrict__ p, int H) {
    if constexpr (kVec) {
        const int i0 = threadIdx.x * kRegs;
        if (i0 < H) {
            const float4 a = *reinterpret_cast<const float4*>(p + i0), b = *reinterpret_cast<const float4*>(p + i0 + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int k = 0; k < kRegs; ++k) v[k] = 0.0f;
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRegs; ++k) {
            const int i = reg_index<false>(k);
            v[k] = i < H ? p[i] : 0.0f;
        }
    }
}

template <bool kVec>
__device__ __forceinline__ void load_row(float (&v)[kRegs], const bf16* __restrict__ p, int H) {
    if constexpr (kVec) {
        const int i0 = threadIdx.x * kRegs;
        if (i0 < H) {
            const uint4 a = *reinterpret_cast<const uint4*>(p + i0);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(h[k]);
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < kRegs; ++k) v[k] = 0.0f;
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRegs; ++k) {
            const int i = reg_index<false>(k);
            v[k] = i < H ? __bfloat162float(p[i]) : 0.0f;
        }
    }
}

template <bool kVec>
__device__ __forceinline__ void store_row(float* __restrict__ p, const float (&v)[kRegs], int H) {
    if constexpr (kVec) {
        const int i0 = threadIdx.x * kRegs;
        if (i0 < H) {
            *reinterpret_cast<float4*>(p + i0) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(p + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRegs; ++k) {
            const int i = reg_index<false>(k);
            if (i < H) p[i] = v[k];
        }
    }
}

template <bool kVec>
__device__ __forceinline__ void store_row(bf16* __restrict__ p, const float (&v)[kRegs], int H) {
    if constexpr (kVec) {
        const int i0 = threadIdx.x * kRegs;
        if (i0 < H) {
            uint4 a;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
            for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
            *reinterpret_cast<uint4*>(p + i0) = a;
        }
    } else {
#pragma unroll
        for (int k = 0; k < kRegs; ++k) {
            const int i = reg_index<false>(k);
            if (i < H) p[i] = __float2bfloat16_rn(v[k]);
        }
    }
}

// (v - mean) * rinv * w for the thread's elements; mean 0 if not centered
template <bool kVec>
__device__ __forceinline__ void row_norm(float (&dst)[kRegs], const float (&v)[kRegs], const float* __restrict__ w, int centered, float eps, int H,
                                         float* scratch) {
    if (centered == kScaleOnly) {                       // (the same for every thread of the block: no barrier is skipped by some)
        float wv[kRegs];
        load_row<kVec>(wv, w, H);
#pragma unroll
        for (int k = 0; k < kRegs; ++k) dst[k] = v[k] * wv[k];
        return;
    }
    const float inv_h = 1.0f / (float)H;
    float mean = 0.0f;
    if (centered) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < kRegs; ++k) s += v[k];
        mean = block_sum(s, scratch) * inv_h;
    }
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < kRegs; ++k) {
        const float d = reg_index<kVec>(k) < H ? v[k] - mean : 0.0f;
        q = fmaf(d, d, q);
    }
    const float rinv = 1.0f / sqrtf(block_sum(q, scratch) * inv_h + eps);
    float wv[kRegs];
    load_row<kVec>(wv, w, H);
#pragma unroll
    for (int k = 0; k < kRegs; ++k) dst[k] = (v[k] - mean) * rinv * wv[k];
}

template <typename T, bool kVec>
__global__ void norm_add_norm_regs_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ w_post, int post_centered,
                                          float eps_post, const float* __restrict__ w_next, int next_centered, float eps_next,
                                          T* __restrict__ out, const int* __restrict__ rows, int n_src, int H,
                                          const int* __restrict__ y_places, int y_top, const float* __restrict__ y_weights) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src = r;
    if (rows) {
        src = rows[r];
        if (src < 0 || src >= n_src) src = 0;
    }
    float* xr = x + (size_t)src * H;
    float xv[kRegs];
    load_row<kVec>(xv, xr, H);
    if (y) {
        float yv[kRegs];
        if (y_places) {
            // the sublayer's output for this token is a sum of rows that lie elsewhere (a token's experts), taken in float
            // in the order of the list
#pragma unroll
            for (int k = 0; k < kRegs; ++k) yv[k] = 0.0f;
            for (int j = 0; j < y_top; ++j) {
                float part[kRegs];
                load_row<kVec>(part, y + (size_t)y_places[(size_t)r * y_top + j] * H, H);
                const float f = y_weights ? y_weights[(size_t)r * y_top + j] : 1.0f;
#pragma unroll
                for (int k = 0; k < kRegs; ++k) yv[k] = fmaf(f, part[k], yv[k]);
            }
        } else {
            load_row<kVec>(yv, y + (size_t)r * H, H);
        }
        if (w_post) {
            float nv[kRegs];
            row_norm<kVec>(nv, yv, w_post, post_centered, eps_post, H, scratch);
#pragma unroll
            for (int k = 0; k < kRegs; ++k) xv[k] += nv[k];
        } else {
#pragma unroll
            for (int k = 0; k < kRegs; ++k) xv[k] += yv[k];
        }
        store_row<kVec>(xr, xv, H);
    }
    if (w_next) {
        float nv[kRegs];
        row_norm<kVec>(nv, xv, w_next, next_centered, eps_next, H, scratch);
        store_row<kVec>(out + (size_t)r * H, nv, H);
    } else if (out) {
        store_row<kVec>(out + (size_t)r * H, xv, H);        // the row as it is, in the run dtype
    }
}

__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, long long n, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += row[i % H];
}

template <typename T>
__global__ void rmsnorm_cols_kernel(const T* __restrict__ in, int ld_in, int col, int n, int width, const float* __restrict__ w, float eps,
                                    T* __restrict__ out, int ld_out, int col_a, int col_b) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* v = in + (size_t)blockIdx.x * ld_in + col;
    float q = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float a = to_float(v[i]);
        q = fmaf(a, a, q);
    }
    q = block_sum(q, scratch);
    const float rinv = 1.0f / sqrtf(q / (float)width + eps);
    T* o = out + (size_t)blockIdx.x * ld_out;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const T r = from_float<T>(to_float(v[i]) * rinv * w[i]);
        o[col_a + i] = r;
        if (col_b >= 0) o[col_b + i] = r;
    }
}

}  // namespace

// y (may be NULL): [R, H] in the run dtype; w_post (may be NULL: x += y); w_next (may be NULL: no norm; out then takes the
// row as it is, if out is given); rows (may
// be NULL; only without y): out[r] = next(x[rows[r]]).  x is [n_src, H] float and is changed in place when y is given.
// y_places (may be NULL; H up to 8,192): token r's y is the sum over j < y_top of y[y_places[r y_top + j]] (times
// y_weights[r y_top + j] if given), summed in float in that order: the combine of a mixture of experts, not written out.
LI_EXPORT int li_norm_add_norm(float* x, const void* y, int dtype, const float* w_post, int post_centered, float eps_post, const float* w_next,
                               int next_centered, float eps_next, void* out, const int* rows, int R, int n_src, int H, const int* y_places,
                               int y_top, const float* y_weights, cudaStream_t stream) {
    LI_REQUIRE(y_places == nullptr || (y != nullptr && y_top > 0 && H <= 8 * 1024), "norm_add_norm: a sum of rows needs the rows, a count and at most 8192 columns");
    LI_REQUIRE(R >= 0 && H > 0 && n_src >= 0, "norm_add_norm: bad sizes R=%d H=%d", R, H);
    LI_REQUIRE(y == nullptr || rows == nullptr, "norm_add_norm: gathered rows cannot take a sublayer's output");
    LI_REQUIRE(w_next == nullptr || out != nullptr, "norm_add_norm: a following norm needs an output");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "norm_add_norm: unknown dtype %d", dtype);
    if (R == 0) return 0;
    cudaError_t e;
    if (H <= kRegs * 1024) {
        // the row in registers: as few threads as hold it, a multiple of 32, at least 64
        int threads = ((ceil_div(H, kRegs) + 31) / 32) * 32;
        if (threads < 64) threads = 64;
        // 16-byte moves where every row starts on such a boundary
        const bool vec = H % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                         ((uintptr_t)w_post % 16) == 0 && ((uintptr_t)w_next % 16) == 0;
#define LI_NORM_LAUNCH(TT, VEC)                                                                                                                  \
    e = li_launch_pdl(norm_add_norm_regs_kernel<TT, VEC>, dim3(R), dim3(threads), 0, stream, x, (const TT*)y, w_post, post_centered, eps_post, w_next, \
                      next_centered, eps_next, (TT*)out, rows, n_src, H, y_places, y_top, y_weights)
        if (dtype == LI_F32) {
            if (vec) LI_NORM_LAUNCH(float, true);
            else LI_NORM_LAUNCH(float, false);
        } else {
            if (vec) LI_NORM_LAUNCH(bf16, true);
            else LI_NORM_LAUNCH(bf16, false);
        }
#undef LI_NORM_LAUNCH
        if (e != cudaSuccess) return li_fail("norm_add_norm: launch failed: %s", cudaGetErrorString(e));
        return li_check_launch("norm_add_norm");
    }
    const int threads = 512;
    if (dtype == LI_F32)
        e = li_launch_pdl(norm_add_norm_kernel<float>, dim3(R), dim3(threads), 0, stream, x, (const float*)y, w_post, post_centered, eps_post,
                          w_next, next_centered, eps_next, (float*)out, rows, n_src, H);
    else
        e = li_launch_pdl(norm_add_norm_kernel<bf16>, dim3(R), dim3(threads), 0, stream, x, (const bf16*)y, w_post, post_centered, eps_post,
                          w_next, next_centered, eps_next, (bf16*)out, rows, n_src, H);
    if (e != cudaSuccess) return li_fail("norm_add_norm: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("norm_add_norm");
}

LI_EXPORT int li_add_row(float* x, const float* row, int T, int H, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && H > 0, "add_row: bad sizes");
    if (T == 0) return 0;
    const long long n = (long long)T * H;
    const cudaError_t e = li_launch_pdl(add_row_kernel, dim3((unsigned)ceil_div_ll(n, 256)), dim3(256), 0, stream, x, row, n, H);
    if (e != cudaSuccess) return li_fail("add_row: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("add_row");
}

// in [T, ld_in]: columns col .. col + n - 1 are normalised (the mean of squares taken over `width` elements: n, or fewer
// when the last columns are padding that holds zeros) and written to out [T, ld_out] at col_a and, if col_b >= 0, at col_b.
LI_EXPORT int li_rmsnorm_cols(const void* in, int dtype, int ld_in, int col, int n, int width, const float* w, float eps, void* out, int ld_out,
                              int col_a, int col_b, int T, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && n > 0 && width > 0 && width <= n && col >= 0 && col + n <= ld_in, "rmsnorm_cols: bad columns");
    LI_REQUIRE(col_a >= 0 && col_a + n <= ld_out && col_b + n <= ld_out, "rmsnorm_cols: bad output columns");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "rmsnorm_cols: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const int threads = n >= 512 ? 256 : 128;
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(rmsnorm_cols_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)in, ld_in, col, n, width, w, eps, (float*)out,
                          ld_out, col_a, col_b);
    else
        e = li_launch_pdl(rmsnorm_cols_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)in, ld_in, col, n, width, w, eps, (bf16*)out,
                          ld_out, col_a, col_b);
    if (e != cudaSuccess) return li_fail("rmsnorm_cols: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("rmsnorm_cols");
}
