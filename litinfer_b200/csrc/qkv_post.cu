// What may stand between the q|k|v product and attention, as one kernel:
//
//   1. a short causal convolution over time on every channel of q, k and v (no bias, no activation):
//        u'_t[c] = sum_j w[c][j] u_(t - taps + 1 + j)[c],
//      inputs before a sequence's portion come from the request's state (the last taps - 1 projected rows, oldest
//      first), zeros before the sequence's start (a cleared state);
//   2. an RMS norm per head on queries and keys, with a weight of head size shared by the heads;
//   3. the rotation of the first rotary_dim elements of each query and key head (pair j with j + rotary_dim / 2,
//      angle float(pos) / denom[j]);
//   4. q written to `out` (the q columns of a [T, (nh + 2 nkv) dh] row), k and v into the paged cache (values transposed).
//
// Each step is optional (no convolution weights, null norm weights, rotary_dim 0).  One warp per (token, head of q|k|v); the head's
// elements stay in registers, the rotation's partners meet through shared memory.  Convolution, norm and angles are
// computed in float from run-dtype inputs and rounded once.  The state itself is moved on by li_conv_state_shift.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kPerLane = 16;        // head_dim <= 512

// TAPS: the taps at compile time (their loads are then all in flight at once), or 0: any number, at run time.
// PER: elements of a head a lane holds (4: heads of up to 128; 16: up to 512); the loops over them are unrolled, and the
// short form has a third of the instructions and registers of the long one.
template <typename T, int TAPS, int PER>
__global__ void __launch_bounds__(kWarps * 32)
conv_norm_rope_kv_kernel(const T* __restrict__ proj, T* __restrict__ out, const float* __restrict__ conv_w, int taps_rt,
                         float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ q_start,
                         const int* __restrict__ seq_of_token, const int* __restrict__ slots, const float* __restrict__ q_norm,
                         const float* __restrict__ k_norm, float eps, int norm_width, const float* __restrict__ row_rinv,
                         const int* __restrict__ positions,
                         const float* __restrict__ denom, int rotary_dim, const int* __restrict__ slot_mapping, T* __restrict__ kcache,
                         T* __restrict__ vcache, int total, int nh, int nkv, int dh, int page_size, int num_pages, int write, int shift, int to_cache,
                         int out_ld) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int taps = TAPS > 0 ? TAPS : taps_rt;
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * kWarps + warp_in_block;
    if (unit >= total) return;
    const int heads = nh + 2 * nkv;
    const int t = unit / heads, head = unit - t * heads;
    const int N = heads * dh;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    if (!is_q && !write) return;
    const int c0 = head * dh;
    const int per = (dh + 31) >> 5;
    float v[PER];
    // 1. the convolution (or the plain value)
    if (conv_w != nullptr) {
        const int s = seq_of_token[t];
        const int q0 = q_start[s];
        const int li = t - q0;
        float* st = taps > 1 ? state + (size_t)slots[s] * state_stride + state_off : nullptr;      // one tap reads no older row
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            float acc = 0.0f;
            if (i < per && d < dh) {
                const int c = c0 + d;
#pragma unroll
                for (int j = 0; j < (TAPS > 0 ? TAPS : taps); ++j) {
                    const int src = li - (taps - 1) + j;
                    const float u = src >= 0 ? to_float(proj[(size_t)(q0 + src) * N + c]) : st[(size_t)(taps - 1 + src) * N + c];
                    acc = fmaf(conv_w[(size_t)c * taps + j], u, acc);
                }
                if (shift && taps > 1) {
                    // a step of single tokens: nobody else reads this channel of this sequence's state, so it moves on here
                    // (oldest first; the newest row is the token's own projection)
                    for (int j = 0; j + 1 < taps; ++j)
                        st[(size_t)j * N + c] = j + 2 < taps ? st[(size_t)(j + 1) * N + c] : to_float(proj[(size_t)t * N + c]);
                }
            }
            v[i] = acc;
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            v[i] = (i < per && d < dh) ? to_float(proj[(size_t)t * N + c0 + d]) : 0.0f;
        }
    }
    // 2. the norm of a query or key head
    const float* nw = is_q ? q_norm : (is_k ? k_norm : nullptr);
    if (nw && row_rinv) {
        // a norm over the whole projection: the factor was taken over all heads, the weight is per channel
        const float rinv = row_rinv[2 * (size_t)t + (is_q ? 0 : 1)];
        const float* wc = nw + (is_q ? c0 : c0 - nh * dh);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) v[i] = v[i] * rinv * wc[d];
        }
    } else if (nw) {
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) q = fmaf(v[i], v[i], q);
        q = warp_sum(q);
        const float rinv = 1.0f / sqrtf(q / (float)norm_width + eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) v[i] = v[i] * rinv * nw[d];
        }
    }
    // 3. the rotation
    if (rotary_dim > 0 && (is_q || is_k)) {
        float* sh = smem + (size_t)warp_in_block * dh;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) sh[d] = v[i];
        }
        __syncwarp();
        const int half = rotary_dim >> 1;
        const float pos = (float)positions[t];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < rotary_dim) {
                const int j = d < half ? d : d - half;
                float sn, cs;
                sincosf(pos / denom[j], &sn, &cs);
                const float a = sh[j], b = sh[j + half];
                v[i] = d < half ? a * cs - b * sn : b * cs + a * sn;
            }
        }
    }
    // 4. where it goes (keys and values of a long step stay in the row: a kernel that writes whole pieces of pages takes them from there)
    if (is_q || !to_cache) {
        T* o = out + (size_t)t * out_ld + c0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) o[d] = from_float<T>(v[i]);
        }
        return;
    }
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot - page * page_size;
    if (slot < 0 || page >= num_pages) return;              // validated on the host; never write outside the cache
    if (is_k) {
        T* dst = kcache + (((size_t)page * nkv + (head - nh)) * page_size + off) * dh;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) dst[d] = from_float<T>(v[i]);
        }
    } else {
        T* dst = vcache + ((size_t)page * nkv + (head - nh - nkv)) * dh * page_size + off;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) dst[(size_t)d * page_size] = from_float<T>(v[i]);
        }
    }
}

// One block per token: the reciprocal root of the mean of squares over up to two ranges of columns.
template <typename T>
__global__ void row_rinv_kernel(const T* __restrict__ x, int ld, int col0, int n0, int width0, int col1, int n1, int width1, float eps,
                                float* __restrict__ out) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* row = x + (size_t)blockIdx.x * ld;
    float a = 0.0f, b = 0.0f;
    for (int i = threadIdx.x; i < n0; i += blockDim.x) {
        const float v = to_float(row[col0 + i]);
        a = fmaf(v, v, a);
    }
    for (int i = threadIdx.x; i < n1; i += blockDim.x) {
        const float v = to_float(row[col1 + i]);
        b = fmaf(v, v, b);
    }
    a = block_sum(a, scratch);
    __syncthreads();
    b = block_sum(b, scratch);
    if (threadIdx.x == 0) {
        out[2 * (size_t)blockIdx.x] = 1.0f / sqrtf(a / (float)width0 + eps);
        out[2 * (size_t)blockIdx.x + 1] = n1 > 0 ? 1.0f / sqrtf(b / (float)width1 + eps) : 0.0f;
    }
}

// The same with a warp per token, eight tokens a block, and loads of 16 bytes: for rows, ranges and columns that are
// multiples of a load's elements (8 of bfloat16, 4 of float).  No barrier; a lane sums its loads in order, then the lanes.
template <typename T>
__global__ void __launch_bounds__(256)
row_rinv_warp_kernel(const T* __restrict__ x, int ld, int col0, int n0, int width0, int col1, int n1, int width1, float eps,
                     float* __restrict__ out, int rows) {
    constexpr int V = 16 / (int)sizeof(T);
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* row = x + (size_t)r * ld;
    float sums[2] = {0.0f, 0.0f};
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const T* p = row + (which ? col1 : col0);
        const int n = which ? n1 : n0;
        float s = 0.0f;
        for (int i = V * lane; i < n; i += 32 * V) {
            const uint4 u = *reinterpret_cast<const uint4*>(p + i);
            if constexpr (sizeof(T) == 2) {
                const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float lo = __uint_as_float(w[k] << 16), hi = __uint_as_float(w[k] & 0xffff0000u);
                    s = fmaf(lo, lo, s);
                    s = fmaf(hi, hi, s);
                }
            } else {
                const float f[4] = {__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w)};
#pragma unroll
                for (int k = 0; k < 4; ++k) s = fmaf(f[k], f[k], s);
            }
        }
        sums[which] = warp_sum(s);
    }
    if (lane == 0) {
        out[2 * (size_t)r] = 1.0f / sqrtf(sums[0] / (float)width0 + eps);
        out[2 * (size_t)r + 1] = n1 > 0 ? 1.0f / sqrtf(sums[1] / (float)width1 + eps) : 0.0f;
    }
}

}  // namespace

LI_EXPORT int li_row_rinv(const void* x, int dtype, int ld, int col0, int n0, int width0, int col1, int n1, int width1, float eps, float* out,
                          int T, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && n0 > 0 && width0 > 0 && col0 >= 0 && col0 + n0 <= ld, "row_rinv: bad first range");
    LI_REQUIRE(n1 >= 0 && (n1 == 0 || (width1 > 0 && col1 >= 0 && col1 + n1 <= ld)), "row_rinv: bad second range");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "row_rinv: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const int threads = n0 + n1 >= 1024 ? 256 : 128;
    cudaError_t e;
    const int vec = dtype == LI_F32 ? 4 : 8;
    if (ld % vec == 0 && col0 % vec == 0 && n0 % vec == 0 && col1 % vec == 0 && n1 % vec == 0 && (uintptr_t)x % 16 == 0) {
        const dim3 grid((unsigned)((T + 7) / 8));
        if (dtype == LI_F32)
            e = li_launch_pdl(row_rinv_warp_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ld, col0, n0, width0, col1, n1, width1, eps, out, T);
        else
            e = li_launch_pdl(row_rinv_warp_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ld, col0, n0, width0, col1, n1, width1, eps, out, T);
        if (e != cudaSuccess) return li_fail("row_rinv: launch failed: %s", cudaGetErrorString(e));
        return li_check_launch("row_rinv");
    }
    if (dtype == LI_F32)
        e = li_launch_pdl(row_rinv_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)x, ld, col0, n0, width0, col1, n1, width1, eps, out);
    else
        e = li_launch_pdl(row_rinv_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)x, ld, col0, n0, width0, col1, n1, width1, eps, out);
    if (e != cudaSuccess) return li_fail("row_rinv: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("row_rinv");
}

// proj, out: [T, (nh + 2 nkv) dh] in the run dtype (out may not be proj when taps > 1: tokens read their neighbours' rows).
// conv_w [(nh + 2 nkv) dh, taps] float (NULL: no convolution; one tap: a factor per channel, no state); state [slots, state_stride] float with the
// convolution's rows at state_off; q_norm, k_norm [dh] float (NULL: no norm), the mean of squares over norm_width
// elements (dh, or fewer when heads are padded with zeros); rotary_dim 0: no rotation.  write 0: only q is made.
// to_cache 0: keys and values go to their columns of `out` instead of the cache (li_rope_kv_write with rotary_dim 0 stores them).
// row_rinv [T, 2] (may be NULL): the norm is over the whole projection of q and of k (li_row_rinv made the factors), and
// q_norm [nh dh], k_norm [nkv dh] are weights per channel.  nkv 0 (write 0): proj holds queries only.  out_ld: elements
// of a row of out (0: as many as proj's), so that queries alone can be written into rows that attention reads as q|k|v.
// shift: the caller promises that every sequence of the step has one token; the state then moves on in this launch
// (with write 0 it does not move at all: the entry that writes the cache moves it).
LI_EXPORT int li_conv_norm_rope_kv(const void* proj, void* out, int dtype, const float* conv_w, int taps, float* state,
                                   long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
                                   const float* q_norm, const float* k_norm, float eps, int norm_width, const float* row_rinv,
                                   const int* positions, const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh,
                                   int page_size, int num_pages, int write, int shift, int to_cache, int out_ld, cudaStream_t stream) {
    if (out_ld == 0) out_ld = (nh + 2 * nkv) * dh;
    LI_REQUIRE(out_ld >= (nh + 2 * nkv) * dh, "conv_norm_rope_kv: output rows of %d elements are too short", out_ld);
    LI_REQUIRE(T >= 0 && nh > 0 && nkv >= 0 && dh > 0 && page_size > 0, "conv_norm_rope_kv: bad sizes");
    LI_REQUIRE(nkv > 0 || !write, "conv_norm_rope_kv: keys and values are to be written, and there are none");
    LI_REQUIRE(dh <= 32 * kPerLane, "conv_norm_rope_kv: head_dim %d is larger than %d", dh, 32 * kPerLane);
    LI_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= dh, "conv_norm_rope_kv: rotary_dim %d must be even and at most head_dim %d",
               rotary_dim, dh);
    LI_REQUIRE(rotary_dim == 0 || denom != nullptr, "conv_norm_rope_kv: rotary_dim %d without denominators", rotary_dim);
    LI_REQUIRE(taps >= 1 && (taps == 1 || (conv_w != nullptr && state != nullptr && proj != out)),
               "conv_norm_rope_kv: a convolution over %d taps needs weights, a state and an output of its own", taps);
    LI_REQUIRE((q_norm == nullptr) == (k_norm == nullptr) || nkv == 0, "conv_norm_rope_kv: queries and keys are normalised together or not at all");
    LI_REQUIRE(row_rinv == nullptr || q_norm != nullptr, "conv_norm_rope_kv: a norm over the whole projection needs its weights");
    LI_REQUIRE(norm_width > 0 && norm_width <= dh, "conv_norm_rope_kv: bad norm width %d", norm_width);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "conv_norm_rope_kv: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const long long total = (long long)T * (nh + 2 * nkv);
    LI_REQUIRE(total < (1LL << 31), "conv_norm_rope_kv: too many (token, head) pairs");
    const dim3 grid((unsigned)ceil_div_ll(total, kWarps));
    const size_t smem = (size_t)kWarps * dh * sizeof(float);
    cudaError_t e;
#define LI_CONV_LAUNCH(TT, TAPS_)                                                                                                             \
    e = li_launch_pdl(dh <= 128 ? conv_norm_rope_kv_kernel<TT, TAPS_, 4> : conv_norm_rope_kv_kernel<TT, TAPS_, kPerLane>, grid, dim3(kWarps * 32), smem, stream, (const TT*)proj, (TT*)out, conv_w, taps, state, \
                      state_stride, state_off, q_start, seq_of_token, slots, q_norm, k_norm, eps, norm_width, row_rinv, positions, denom, rotary_dim, \
                      slot_mapping, (TT*)kcache, (TT*)vcache, (int)total, nh, nkv, dh, page_size, num_pages, write, (shift && write) ? 1 : 0, to_cache, out_ld)
#define LI_CONV_TAPS(TT)                         \
    switch (conv_w ? taps : 1) {                 \
        case 1: LI_CONV_LAUNCH(TT, 1); break;    \
        case 2: LI_CONV_LAUNCH(TT, 2); break;    \
        case 3: LI_CONV_LAUNCH(TT, 3); break;    \
        case 4: LI_CONV_LAUNCH(TT, 4); break;    \
        default: LI_CONV_LAUNCH(TT, 0); break;   \
    }
    if (dtype == LI_F32) {
        LI_CONV_TAPS(float)
    } else {
        LI_CONV_TAPS(bf16)
    }
#undef LI_CONV_TAPS
#undef LI_CONV_LAUNCH
    if (e != cudaSuccess) return li_fail("conv_norm_rope_kv: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("conv_norm_rope_kv");
}

// Latent attention with a rotated part: what stands between its projections and attention over the latent.
// Per token, with a latent of R and a rotated part of dr elements, heads of the attention dl >= R + dr wide:
//   * the key/value latent  c = low[col_c : col_c + R] / sqrt(mean(.^2) + eps) * w  goes to the key head's and the value head's
//     first R columns of the attention row `out` [T, (nh + 2) dl];
//   * the one rotated key part all heads share, low[col_r : col_r + dr], is rotated and follows c in the key head;
//   * every query head's rotated part, q[h (d + dr) + d : (h + 1) (d + dr)], is rotated and goes behind the head's first R
//     columns (which the product that carries the unrotated query into the latent space fills);
//   * what is left of every head (and of the value head behind c) is set to zero.
// Rotation: pair i turns by float(pos) / denom[i]; `interleaved`: the pair is (2i, 2i + 1), else (i, i + dr / 2); cosine and
// sine are multiplied by `magnitude`.  Norm and angles in float, one rounding.  One block per token.
namespace {
template <typename T>
__global__ void latent_rope_post_kernel(const T* __restrict__ low, int ld_low, int col_c, int col_r, const T* __restrict__ q, int ld_q, int d,
                                        const float* __restrict__ w, float eps, const int* __restrict__ positions, const float* __restrict__ denom,
                                        float magnitude, int interleaved, T* __restrict__ out, int nh, int R, int dr, int dl) {
    __shared__ float scratch[32];
    extern __shared__ float cs[];                       // [dr / 2][2]: cosine and sine of the token's pairs, with the magnitude
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = dr >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, c;
        sincosf(pos / denom[i], &sn, &c);
        cs[2 * i] = c * magnitude;
        cs[2 * i + 1] = sn * magnitude;
    }
    const T* lrow = low + (size_t)t * ld_low;
    T* orow = out + (size_t)t * (nh + 2) * dl;
    float ssq = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_float(lrow[col_c + i]);
        ssq = fmaf(v, v, ssq);
    }
    ssq = block_sum(ssq, scratch);                      // (its barriers also make the table above visible)
    const float rinv = 1.0f / sqrtf(ssq / (float)R + eps);
    T* khead = orow + (size_t)nh * dl;
    T* vhead = khead + dl;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const T c = from_float<T>(to_float(lrow[col_c + i]) * rinv * w[i]);
        khead[i] = c;
        vhead[i] = c;
    }
    for (int i = R + threadIdx.x; i < dl; i += blockDim.x) vhead[i] = from_float<T>(0.0f);
    // heads 0 .. nh - 1: the queries' rotated parts; head nh: the key's
    for (int idx = threadIdx.x; idx < (nh + 1) * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const T* src = h < nh ? q + (size_t)t * ld_q + (size_t)h * (d + dr) + d : lrow + col_r;
        T* dst = orow + (size_t)h * dl + R;
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float a = to_float(src[ia]), b = to_float(src[ib]);
        const float c = cs[2 * i], sn = cs[2 * i + 1];
        dst[ia] = from_float<T>(a * c - b * sn);
        dst[ib] = from_float<T>(b * c + a * sn);
    }
    const int pad = dl - R - dr;
    for (int idx = threadIdx.x; idx < (nh + 1) * pad; idx += blockDim.x) {
        const int h = idx / pad, i = idx - h * pad;
        orow[(size_t)h * dl + R + dr + i] = from_float<T>(0.0f);
    }
}
}  // namespace

LI_EXPORT int li_latent_rope_post(const void* low, int dtype, int ld_low, int col_c, int col_r, const void* q, int ld_q, int d, const float* w, float eps,
                                  const int* positions, const float* denom, float magnitude, int interleaved, void* out, int T, int nh, int R, int dr,
                                  int dl, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && nh > 0 && R > 0 && dr >= 0 && dr % 2 == 0 && dl >= R + dr && d >= 0, "latent_rope_post: bad sizes nh=%d R=%d dr=%d dl=%d", nh, R, dr, dl);
    LI_REQUIRE(col_c >= 0 && col_c + R <= ld_low && col_r >= 0 && col_r + dr <= ld_low && nh * (d + dr) <= ld_q, "latent_rope_post: columns do not fit the rows");
    LI_REQUIRE(dr == 0 || denom != nullptr, "latent_rope_post: a rotated part needs its denominators");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "latent_rope_post: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const size_t smem = (size_t)(dr > 0 ? dr : 2) * sizeof(float);
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(latent_rope_post_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)low, ld_low, col_c, col_r, (const float*)q, ld_q, d, w,
                          eps, positions, denom, magnitude, interleaved, (float*)out, nh, R, dr, dl);
    else
        e = li_launch_pdl(latent_rope_post_kernel<bf16>, dim3(T), dim3(128), smem, stream, (const bf16*)low, ld_low, col_c, col_r, (const bf16*)q, ld_q, d, w,
                          eps, positions, denom, magnitude, interleaved, (bf16*)out, nh, R, dr, dl);
    if (e != cudaSuccess) return li_fail("latent_rope_post: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("latent_rope_post");
}
