// Mixers that carry a state of fixed size per request instead of a cache that grows: the plain kernels.
//
// Every kernel here finds a sequence's tokens through q_start[s] .. q_start[s + 1] and its state through
// state_slots[s], both on the device, so a step of single tokens launches the same grid whatever the slots hold and can
// be replayed from a captured graph.  A sequence's tokens are walked in order; the state is read once, kept in registers
// and written once.  State, decays, step sizes, gates of the recurrence and every sum are float;
// the projections come in the run dtype.
//
//   * li_causal_conv_silu / li_conv_state_shift: a depthwise causal convolution over the last `taps` inputs of each
//     channel followed by x / (1 + exp(-x)); the taps - 1 inputs before a portion come from the state, which the
//     second kernel then moves on (two launches: every token of the step reads the old state).
//   * li_ssm_scan: per head a state S [N, P]:  S = exp(-exp(A_log) dt) S + dt B x^T,  y = S^T C + D x, with
//     dt = softplus(dt_raw + dt_bias) per token and head, B and C shared by the heads of a group.
//   * li_decay_scan: per head a state S [d, dv]:  S = decay S + k v^T,  o = S^T q, with q, k, v passed through
//     x / (1 + exp(-x)) on the way in.
//   * li_gla_scan: per head a state S [d, dv] with a decay per token and key channel:  S = diag(a_t) S + k v^T,
//     o = S^T (q / sqrt(d)),  a_t = sigmoid(z_t)^(1 / tau) from float logits z.
//   * li_delta_prepare / li_delta_scan: per head a state S [d, dv] under the gated delta rule with a decay per token and key
//     channel:  S = diag(g) S,  u = beta (v - S^T k),  S = S + k u^T,  o = S^T q; the first kernel makes what does not depend on
//     the state (convolution, unit vectors q and k, decays, beta), the second walks.
//   * li_channel_scan: a state S [N] per channel c with a decay per token, channel and element:
//     S = exp(dt_c A[c, :]) S + dt_c x_c B,  y_c = (S . C + D_c x_c) silu(z_c),  dt = softplus(dt_raw), A = -exp(A_log).
//   * li_gated_rmsnorm: RMSNorm in equal groups of a float row, with a gate before the norm (y * silu(z)) or after
//     it (norm(y) * sigmoid(g), or norm(y) * silu(g)).
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

constexpr int kMaxTaps = 8;

// in: [T, in_stride] with the C channels at column in_off; w [C, taps] (the last tap is the current token's), b [C];
// state [slots, state_stride] with the last taps - 1 inputs at state_off, oldest first, [taps - 1, C].
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int in_stride, int in_off, const float* __restrict__ w, const float* __restrict__ b,
                                        float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ q_start,
                                        const int* __restrict__ seq_of_token, const int* __restrict__ slots, T* __restrict__ out, int C, int taps,
                                        int shift) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_of_token[t];
    const int q0 = q_start[s];
    const int li = t - q0;
    float* st = state + (size_t)slots[s] * state_stride + state_off;
    float acc = b[c];
    for (int k = 0; k < taps; ++k) {
        const int i = li - (taps - 1) + k;
        const float v = i >= 0 ? to_float(in[(size_t)(q0 + i) * in_stride + in_off + c]) : st[(size_t)(taps - 1 + i) * C + c];
        acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    out[(size_t)t * C + c] = from_float<T>(silu_f(acc));
    if (shift) {
        // a step of single tokens: nobody else reads this sequence's state, so it moves on here (oldest first)
        for (int j = 0; j + 1 < taps; ++j)
            st[(size_t)j * C + c] = j + 2 < taps ? st[(size_t)(j + 1) * C + c] : to_float(in[(size_t)t * in_stride + in_off + c]);
    }
}

template <typename T>
__global__ void conv_state_shift_kernel(const T* __restrict__ in, int in_stride, int in_off, float* __restrict__ state, long long state_stride,
                                        long long state_off, const int* __restrict__ q_start, const int* __restrict__ slots, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int q0 = q_start[s], n = q_start[s + 1] - q0;
    if (n <= 0) return;
    float* st = state + (size_t)slots[s] * state_stride + state_off;
    float keep[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < taps - 1) {
            const int i = n - (taps - 1) + j;                    // index among the portion's inputs; negative: an older one
            keep[j] = i >= 0 ? to_float(in[(size_t)(q0 + i) * in_stride + in_off + c]) : st[(size_t)(taps - 1 + i) * C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
        if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
}

// The two recurrences walk a sequence's tokens in order, but every column of a head's state moves on by itself:
// S[:, c] <- a_t S[:, c] + w_t[:] u_t[c],  out_t[c] = sum_i S[i, c] r_t[i].  So a column is the unit of work.  A warp holds
// eight columns in registers, each lane the same few neighbouring elements of all eight, so that one load of w and of r
// from shared memory serves eight columns (with a column per eight lanes the kernel was bound by shared-memory wavefronts
// and by the instructions around them: 127 a warp and token for four columns).  A block, up to 16 warps, stages the vectors
// of kStage tokens that all its columns need (w, r, and the scalars) in shared memory once, with the activations applied.
// The eight sums over the lanes take nine shuffles together.  The state is stored column by column
// ([head][column][element]) so that it is read and written in whole lines.
//
// Long portions are cut into chunks that run side by side (a sequence alone has too few columns to fill the GPU, and a
// walk over thousands of tokens is bound by its latency): `seg` names the chunks (begin, end, chunk, slot) and `mode` says
// which of three passes this is.  kScanLocal: every chunk from a state of zeros, no outputs, its end state to
// chunk_state[chunk].  li_scan_carry then walks each sequence's chunks in order, S <- decay(chunk) S + end state, and
// leaves in chunk_state[chunk] the state the chunk starts from (and the sequence's last state in its slot).  kScanApply:
// every chunk again from that state, with outputs.  Without `seg` (kScanWhole) a sequence is one piece, read from and
// written to its slot: steps of single tokens and short portions.
enum { kScanWhole = 0, kScanLocal = 1, kScanApply = 2 };
constexpr int kStage = 16;          // tokens staged at a time

// One sequence or chunk of it: which tokens, whose slot, which chunk.
struct Piece {
    int q0, q1, slot, chunk;
};
__device__ __forceinline__ Piece piece_of(const int* __restrict__ seg, const int* __restrict__ q_start, const int* __restrict__ slots) {
    Piece p;
    if (seg) {
        const int4 sg = reinterpret_cast<const int4*>(seg)[blockIdx.z];
        p.q0 = sg.x; p.q1 = sg.y; p.chunk = sg.z; p.slot = sg.w;
    } else {
        p.q0 = q_start[blockIdx.z]; p.q1 = q_start[blockIdx.z + 1]; p.slot = slots[blockIdx.z]; p.chunk = 0;
    }
    return p;
}

constexpr int kWarpCols = 8;        // columns a warp walks

// E neighbouring floats of a staged row (E = 1, 2, 4, 8), one load of up to 16 bytes at a time.
template <int E>
__device__ __forceinline__ void load_elements(float (&v)[E], const float* p) {
    if constexpr (E == 1) {
        v[0] = p[0];
    } else if constexpr (E == 2) {
        const float2 a = *reinterpret_cast<const float2*>(p);
        v[0] = a.x; v[1] = a.y;
    } else {
#pragma unroll
        for (int q = 0; q < E / 4; ++q) {
            const float4 a = reinterpret_cast<const float4*>(p)[q];
            v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
        }
    }
}

// Sums over the 32 lanes of eight values a lane: each exchange halves the values a lane still carries, so nine shuffles
// do for all eight.  Afterwards every lane holds the sum of value 4 (lane >> 4 & 1) + 2 (lane >> 3 & 1) + (lane >> 2 & 1).
__device__ __forceinline__ float sum8_across_warp(const float (&a)[8], int lane) {
    float b[4], c[2];
    const bool up16 = lane & 16, up8 = lane & 8, up4 = lane & 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = (up16 ? a[j + 4] : a[j]) + __shfl_xor_sync(0xffffffffu, up16 ? a[j] : a[j + 4], 16);
#pragma unroll
    for (int j = 0; j < 2; ++j) c[j] = (up8 ? b[j + 2] : b[j]) + __shfl_xor_sync(0xffffffffu, up8 ? b[j] : b[j + 2], 8);
    float v = (up4 ? c[1] : c[0]) + __shfl_xor_sync(0xffffffffu, up4 ? c[0] : c[1], 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v + __shfl_xor_sync(0xffffffffu, v, 1);
}
__device__ __forceinline__ int column_after_sum8(int lane) { return 4 * ((lane >> 4) & 1) + 2 * ((lane >> 3) & 1) + ((lane >> 2) & 1); }

// The same for N = 8, 4 or 2 values a lane; the exchanges come in the same order (lanes 16, 8, 4, 2, 1 apart), so a column's sum
// is the same bits whichever N carries it.  column_after_sum<N>: whose sum a lane holds; lane_of_column<N>: the first lane that
// holds a column's; sum_is_first<N>: whether this lane is that one.
template <int N>
__device__ __forceinline__ float sum_across_warp(const float (&a)[N], int lane) {
    if constexpr (N == 8) {
        return sum8_across_warp(a, lane);
    } else if constexpr (N == 4) {
        float b[2];
        const bool up16 = lane & 16, up8 = lane & 8;
#pragma unroll
        for (int j = 0; j < 2; ++j) b[j] = (up16 ? a[j + 2] : a[j]) + __shfl_xor_sync(0xffffffffu, up16 ? a[j] : a[j + 2], 16);
        float v = (up8 ? b[1] : b[0]) + __shfl_xor_sync(0xffffffffu, up8 ? b[0] : b[1], 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        return v + __shfl_xor_sync(0xffffffffu, v, 1);
    } else {
        static_assert(N == 2, "eight, four or two values a lane");
        const bool up16 = lane & 16;
        float v = (up16 ? a[1] : a[0]) + __shfl_xor_sync(0xffffffffu, up16 ? a[0] : a[1], 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        return v + __shfl_xor_sync(0xffffffffu, v, 1);
    }
}
template <int N>
__device__ __forceinline__ int column_after_sum(int lane) {
    if constexpr (N == 8) return column_after_sum8(lane);
    else if constexpr (N == 4) return 2 * ((lane >> 4) & 1) + ((lane >> 3) & 1);
    else return (lane >> 4) & 1;
}
template <int N>
__device__ __forceinline__ int lane_of_column(int j) {
    if constexpr (N == 8) return 16 * ((j >> 2) & 1) + 8 * ((j >> 1) & 1) + 4 * (j & 1);
    else if constexpr (N == 4) return 16 * ((j >> 1) & 1) + 8 * (j & 1);
    else return 16 * (j & 1);
}
template <int N>
__device__ __forceinline__ bool sum_is_first(int lane) { return (lane & (N == 8 ? 3 : N == 4 ? 7 : 15)) == 0; }

// xbc [T, C]: x (heads * P) | B (groups * N) | C (groups * N), after convolution and activation.  E = ceil(N / 32)
// rounded up to 1, 2, 4 or 8 elements a lane; blockDim.x / 32 warps of eight columns each.
template <typename T, int E>
__global__ void __launch_bounds__(512)
ssm_scan_kernel(const T* __restrict__ xbc, int C, const T* __restrict__ dt_raw, int dt_stride, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ D, float* __restrict__ state, long long state_stride,
                const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ y, int heads, int P, int N, int groups,
                const int* __restrict__ seg, int mode, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    constexpr int NP = 32 * E;                         // a staged row, padded with zeros
    const int warps = blockDim.x >> 5, cols = kWarpCols * warps;
    extern __shared__ __align__(16) float smem[];
    float* Bs = smem;                           // [kStage][NP]
    float* Cs = Bs + kStage * NP;               // [kStage][NP]
    float* xs = Cs + kStage * NP;               // [kStage][cols]
    float* dts = xs + kStage * cols;            // [kStage] step size
    float* das = dts + kStage;                  // [kStage] decay
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const Piece pc = piece_of(seg, q_start, slots);
    const int q0 = pc.q0, q1 = pc.q1;
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * cols + warp * kWarpCols;          // this warp's first column of the head
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const size_t head_at = (size_t)h * P * N;
    float* st = state + (size_t)pc.slot * state_stride + head_at;
    float* cst = chunk_state ? chunk_state + (size_t)pc.chunk * heads * P * N + head_at : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[kWarpCols][E];
#pragma unroll
    for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e)
            S[j][e] = (mode != kScanLocal && col0 + j < P && E * lane + e < N) ? from[(size_t)(col0 + j) * N + E * lane + e] : 0.0f;
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = D[h];
    if (mode == kScanLocal && blockIdx.x == 0 && warp == 0) {
        // the chunk's decay as a whole, for the pass that carries states from chunk to chunk
        float sum = 0.0f;
        for (int t = q0 + lane; t < q1; t += 32) sum += -rate * softplus_f(to_float(dt_raw[(size_t)t * dt_stride + h]) + bias);
        sum = warp_sum(sum);
        if (lane == 0) chunk_decay[(size_t)pc.chunk * heads + h] = expf(sum);
    }
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();                                   // the stage before has been used up
        for (int tk = warp; tk < nt; tk += warps) {
            const T* row = xbc + (size_t)(t0 + tk) * C;
            for (int n = lane; n < NP; n += 32) {
                Bs[tk * NP + n] = n < N ? to_float(row[inner + g * N + n]) : 0.0f;
                if (mode != kScanLocal) Cs[tk * NP + n] = n < N ? to_float(row[inner + (groups + g) * N + n]) : 0.0f;
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tk = e / cols, j = e - tk * cols;
            const int c = blockIdx.x * cols + j;
            xs[e] = c < P ? to_float(xbc[(size_t)(t0 + tk) * C + h * P + c]) : 0.0f;
        }
        if (threadIdx.x < nt) {
            const float dt = softplus_f(to_float(dt_raw[(size_t)(t0 + threadIdx.x) * dt_stride + h]) + bias);
            dts[threadIdx.x] = dt;
            das[threadIdx.x] = expf(-rate * dt);
        }
        __syncthreads();
#pragma unroll 2
        for (int tk = 0; tk < nt; ++tk) {
            float b[E], x[kWarpCols];
            load_elements<E>(b, Bs + tk * NP + E * lane);
            load_elements<kWarpCols>(x, xs + tk * cols + warp * kWarpCols);
            const float dt = dts[tk], decay = das[tk];
            if (mode == kScanLocal) {
#pragma unroll
                for (int j = 0; j < kWarpCols; ++j) {
                    const float dx = dt * x[j];
#pragma unroll
                    for (int e = 0; e < E; ++e) S[j][e] = fmaf(decay, S[j][e], b[e] * dx);
                }
                continue;
            }
            float cc[E], acc[kWarpCols];
            load_elements<E>(cc, Cs + tk * NP + E * lane);
#pragma unroll
            for (int j = 0; j < kWarpCols; ++j) {
                const float dx = dt * x[j];
                acc[j] = 0.0f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    S[j][e] = fmaf(decay, S[j][e], b[e] * dx);
                    acc[j] = fmaf(S[j][e], cc[e], acc[j]);
                }
            }
            const float total = sum8_across_warp(acc, lane);
            const int j = column_after_sum8(lane);
            if ((lane & 3) == 0 && col0 + j < P) y[(size_t)(t0 + tk) * inner + h * P + col0 + j] = fmaf(skip, xs[tk * cols + warp * kWarpCols + j], total);
        }
    }
    if (mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (col0 + j < P && E * lane + e < N) to[(size_t)(col0 + j) * N + E * lane + e] = S[j][e];
    }
}

// q, k [T, stride] at columns q_off + h d, k_off + h d; v at v_off + h dv; all before their activation.
template <typename T, int E>
__global__ void __launch_bounds__(512)
decay_scan_kernel(const T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                  float* __restrict__ out, int heads, int d, int dv, const int* __restrict__ seg, int mode, float* __restrict__ chunk_state) {
    constexpr int DP = 32 * E;
    const int warps = blockDim.x >> 5, cols = kWarpCols * warps;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                           // [kStage][DP]
    float* ks = qs + kStage * DP;               // [kStage][DP]
    float* vs = ks + kStage * DP;               // [kStage][cols]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const Piece pc = piece_of(seg, q_start, slots);
    const int q0 = pc.q0, q1 = pc.q1;
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * cols + warp * kWarpCols;
    const size_t head_at = (size_t)h * dv * d;
    float* st = state + (size_t)pc.slot * state_stride + head_at;
    float* cst = chunk_state ? chunk_state + (size_t)pc.chunk * heads * dv * d + head_at : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[kWarpCols][E];
#pragma unroll
    for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e)
            S[j][e] = (mode != kScanLocal && col0 + j < dv && E * lane + e < d) ? from[(size_t)(col0 + j) * d + E * lane + e] : 0.0f;
    const float lam = decay[h];
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();
        for (int tk = warp; tk < nt; tk += warps) {
            const T* row = qkv + (size_t)(t0 + tk) * stride;
            for (int i = lane; i < DP; i += 32) {
                if (mode != kScanLocal) qs[tk * DP + i] = i < d ? silu_f(to_float(row[q_off + h * d + i])) : 0.0f;
                ks[tk * DP + i] = i < d ? silu_f(to_float(row[k_off + h * d + i])) : 0.0f;
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tk = e / cols, j = e - tk * cols;
            const int c = blockIdx.x * cols + j;
            vs[e] = c < dv ? silu_f(to_float(qkv[(size_t)(t0 + tk) * stride + v_off + h * dv + c])) : 0.0f;
        }
        __syncthreads();
#pragma unroll 2
        for (int tk = 0; tk < nt; ++tk) {
            float kk[E], v[kWarpCols];
            load_elements<E>(kk, ks + tk * DP + E * lane);
            load_elements<kWarpCols>(v, vs + tk * cols + warp * kWarpCols);
            if (mode == kScanLocal) {
#pragma unroll
                for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
                    for (int e = 0; e < E; ++e) S[j][e] = fmaf(lam, S[j][e], kk[e] * v[j]);
                continue;
            }
            float qq[E], acc[kWarpCols];
            load_elements<E>(qq, qs + tk * DP + E * lane);
#pragma unroll
            for (int j = 0; j < kWarpCols; ++j) {
                acc[j] = 0.0f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    S[j][e] = fmaf(lam, S[j][e], kk[e] * v[j]);
                    acc[j] = fmaf(S[j][e], qq[e], acc[j]);
                }
            }
            const float total = sum8_across_warp(acc, lane);
            const int j = column_after_sum8(lane);
            if ((lane & 3) == 0 && col0 + j < dv) out[(size_t)(t0 + tk) * heads * dv + h * dv + col0 + j] = total;
        }
    }
    if (mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (col0 + j < dv && E * lane + e < d) to[(size_t)(col0 + j) * d + E * lane + e] = S[j][e];
    }
}

// Linear attention with a decay per token and key channel.  q, k [T, stride] at columns q_off + h d, k_off + h d; v at
// v_off + h dv (no activation); za [T, za_stride] float: the decays' logits at za_off + h d.  a = exp(log sigmoid(z) / tau),
// taken in float while staging; q is multiplied by q_scale there.  Columns, stages and passes as in decay_scan_kernel; the
// chunk's decay is a number per key channel (the product of its tokens' decays, summed as logarithms).
template <typename T, int E>
__global__ void __launch_bounds__(512)
gla_scan_kernel(const T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off, const float* __restrict__ za, int za_stride, int za_off,
                float inv_tau, float q_scale, float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
                const int* __restrict__ slots, float* __restrict__ out, int heads, int d, int dv, const int* __restrict__ seg, int mode,
                float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    constexpr int DP = 32 * E;
    const int warps = blockDim.x >> 5, cols = kWarpCols * warps;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                           // [kStage][DP]
    float* ks = qs + kStage * DP;               // [kStage][DP]
    float* as = ks + kStage * DP;               // [kStage][DP] decays
    float* vs = as + kStage * DP;               // [kStage][cols]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const Piece pc = piece_of(seg, q_start, slots);
    const int q0 = pc.q0, q1 = pc.q1;
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * cols + warp * kWarpCols;
    const size_t head_at = (size_t)h * dv * d;
    float* st = state + (size_t)pc.slot * state_stride + head_at;
    float* cst = chunk_state ? chunk_state + (size_t)pc.chunk * heads * dv * d + head_at : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[kWarpCols][E];
#pragma unroll
    for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e)
            S[j][e] = (mode != kScanLocal && col0 + j < dv && E * lane + e < d) ? from[(size_t)(col0 + j) * d + E * lane + e] : 0.0f;
    // the chunk's decay per key channel, for the pass that carries states from chunk to chunk: the logarithms of its tokens'
    // decays, summed in the order of the tokens from the staged rows (the pass from zeros stages them where q would stand)
    float logsum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const bool sums = mode == kScanLocal && blockIdx.x == 0;
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();
        for (int tk = warp; tk < nt; tk += warps) {
            const T* row = qkv + (size_t)(t0 + tk) * stride;
            const float* zrow = za + (size_t)(t0 + tk) * za_stride + za_off + h * d;
            for (int i = lane; i < DP; i += 32) {
                const float lg = i < d ? -softplus_f(-zrow[i]) * inv_tau : 0.0f;
                qs[tk * DP + i] = mode == kScanLocal ? lg : i < d ? to_float(row[q_off + h * d + i]) * q_scale : 0.0f;
                ks[tk * DP + i] = i < d ? to_float(row[k_off + h * d + i]) : 0.0f;
                as[tk * DP + i] = i < d ? expf(lg) : 0.0f;
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tk = e / cols, j = e - tk * cols;
            const int c = blockIdx.x * cols + j;
            vs[e] = c < dv ? to_float(qkv[(size_t)(t0 + tk) * stride + v_off + h * dv + c]) : 0.0f;
        }
        __syncthreads();
        if (sums) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = threadIdx.x + u * blockDim.x;
                if (i < d)
                    for (int tk = 0; tk < nt; ++tk) logsum[u] += qs[tk * DP + i];
            }
        }
#pragma unroll 2
        for (int tk = 0; tk < nt; ++tk) {
            float kk[E], aa[E], v[kWarpCols];
            load_elements<E>(kk, ks + tk * DP + E * lane);
            load_elements<E>(aa, as + tk * DP + E * lane);
            load_elements<kWarpCols>(v, vs + tk * cols + warp * kWarpCols);
            if (mode == kScanLocal) {
#pragma unroll
                for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
                    for (int e = 0; e < E; ++e) S[j][e] = fmaf(aa[e], S[j][e], kk[e] * v[j]);
                continue;
            }
            float qq[E], acc[kWarpCols];
            load_elements<E>(qq, qs + tk * DP + E * lane);
#pragma unroll
            for (int j = 0; j < kWarpCols; ++j) {
                acc[j] = 0.0f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    S[j][e] = fmaf(aa[e], S[j][e], kk[e] * v[j]);
                    acc[j] = fmaf(S[j][e], qq[e], acc[j]);
                }
            }
            const float total = sum8_across_warp(acc, lane);
            const int j = column_after_sum8(lane);
            if ((lane & 3) == 0 && col0 + j < dv) out[(size_t)(t0 + tk) * heads * dv + h * dv + col0 + j] = total;
        }
    }
    if (sums) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = threadIdx.x + u * blockDim.x;
            if (i < d) chunk_decay[((size_t)pc.chunk * heads + h) * d + i] = expf(logsum[u]);
        }
    }
    if (mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (col0 + j < dv && E * lane + e < d) to[(size_t)(col0 + j) * d + E * lane + e] = S[j][e];
    }
}

// The gated delta rule with a decay per token, head and key channel.  Per head a state S [d, dv]:
//     S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t      (in this order: o sees the write)
// Two kernels.  delta_prepare_kernel makes everything of a token that does not depend on the state, one warp per unit of
// work, in float: for a key head the convolution and silu of its q and k channels, both made unit vectors
// (x / sqrt(sum x^2 + unit_eps), q times q_scale) and k . q; for a head the decays g = exp(-exp(A_log[h]) softplus(za)) and
// beta = sigmoid(b); for a head's values the convolution and silu.  Rows of DP = 32 E floats with zeros behind d, so that the
// scan stages them as they are: prep_qk [T, kv_heads, 2 DP + 4] (q | k | k . q), prep_g [T, heads, DP + 4] (g | beta),
// v [T, heads dv].  Every channel of the convolution belongs to one warp, which also moves the channel's state on in a step of
// single tokens (`shift`).
// TAPS: the taps at compile time (their loads are then all in flight at once), or 0: any number, at run time.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* __restrict__ proj, int stride, int col0, int b_off, const float* __restrict__ conv_w, int taps_rt,
                     float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ q_start,
                     const int* __restrict__ seq_of_token, const int* __restrict__ slots, const float* __restrict__ za, int za_stride, int za_off,
                     const float* __restrict__ A_log, float q_scale, float unit_eps, float* __restrict__ prep_qk, float* __restrict__ prep_g,
                     float* __restrict__ v_out, int total, int heads, int kv_heads, int d, int dv, int DP, int shift) {
    pdl_launch_dependents();
    pdl_wait();
    const int taps = TAPS > 0 ? TAPS : taps_rt;
    const int units = kv_heads + 2 * heads;
    const long long id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= (long long)total * units) return;
    const int t = (int)(id / units), u = (int)(id - (long long)t * units);
    const int lane = threadIdx.x & 31;
    const int s = seq_of_token[t];
    const int q0 = q_start[s], li = t - q0;
    const int C = 2 * kv_heads * d + heads * dv;
    float* st = state + (size_t)slots[s] * state_stride + state_off;
    // channel c of the convolution for this token, with silu; the channel's state moves on if the step is one of single tokens
    auto conv = [&](int c) {
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < (TAPS > 0 ? TAPS : taps); ++k) {
            const int i = li - (taps - 1) + k;
            const float v = i >= 0 ? to_float(proj[(size_t)(q0 + i) * stride + col0 + c]) : st[(size_t)(taps - 1 + i) * C + c];
            acc = fmaf(conv_w[(size_t)c * taps + k], v, acc);
        }
        if (shift)
            for (int j = 0; j + 1 < taps; ++j)
                st[(size_t)j * C + c] = j + 2 < taps ? st[(size_t)(j + 1) * C + c] : to_float(proj[(size_t)t * stride + col0 + c]);
        return silu_f(acc);
    };
    if (u < kv_heads) {
        float qv[8], kv[8];
        float qq = 0.0f, kk = 0.0f, qk = 0.0f;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int i = lane + 32 * it;
            qv[it] = i < d ? conv(u * d + i) : 0.0f;
            kv[it] = i < d ? conv(kv_heads * d + u * d + i) : 0.0f;
            qq = fmaf(qv[it], qv[it], qq); kk = fmaf(kv[it], kv[it], kk); qk = fmaf(qv[it], kv[it], qk);
        }
        qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
        const float fq = q_scale / sqrtf(qq + unit_eps), fk = 1.0f / sqrtf(kk + unit_eps);
        float* row = prep_qk + ((size_t)t * kv_heads + u) * (2 * DP + 4);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int i = lane + 32 * it;
            if (i < DP) {
                row[i] = qv[it] * fq;
                row[DP + i] = kv[it] * fk;
            }
        }
        if (lane == 0) row[2 * DP] = qk * fq * fk;
    } else if (u < kv_heads + heads) {
        const int h = u - kv_heads;
        const float rate = -expf(A_log[h]);
        const float* zrow = za + (size_t)t * za_stride + za_off + h * d;
        float* row = prep_g + ((size_t)t * heads + h) * (DP + 4);
        for (int i = lane; i < DP; i += 32) row[i] = i < d ? expf(rate * softplus_f(zrow[i])) : 0.0f;
        if (lane == 0) row[DP] = sigmoid_f(to_float(proj[(size_t)t * stride + b_off + h]));
    } else {
        const int h = u - kv_heads - heads;
        for (int j = lane; j < dv; j += 32) v_out[(size_t)t * heads * dv + h * dv + j] = conv(2 * kv_heads * d + h * dv + j);
    }
}

// The walk itself.  A column of S moves on by itself here too (u[c] depends on column c alone), so it is the walk of
// gla_scan_kernel: a warp holds WC columns (eight, four or two), each lane E neighbouring key channels of all of them; with few
// sequences and heads the columns are spread over more warps, since a token's chain of instructions is as long as its warp has
// columns.  The two sums over the key channels that a token needs, (gS)^T k and (gS)^T q, are taken together before the write, since S_new^T q = (gS)^T q +
// u (k . q).  A block has few warps (a head's columns are spread over many blocks: the walk is a chain of dependent
// instructions per token, and a multiprocessor issues one warp's chain no faster when it holds sixteen of them) and stages the
// prepared rows of kStage tokens as they are, the next stage's while it walks this one's.  One piece per sequence: the rule is not elementwise in S, so chunks of a portion
// do not run side by side.
// 16 bytes from global to shared memory without passing registers; zeros if not valid
__device__ __forceinline__ void stage16(float* dst, const float* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}

template <int E, int WC>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ prep_qk, const float* __restrict__ prep_g, const float* __restrict__ vin, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ out, int heads,
                  int kv_heads, int d, int dv) {
    constexpr int DP = 32 * E;
    const int warps = blockDim.x >> 5, cols = WC * warps;
    // two buffers of kStage tokens each: the next stage's rows are on their way (asynchronous copies of 16 bytes) while this
    // stage is walked.  A buffer: q [kStage][DP] | k [kStage][DP] | decays [kStage][DP] | v [kStage][cols] | (beta ...) [kStage][4]
    // | (k . q ...) [kStage][4]
    extern __shared__ __align__(16) float smem[];
    const int buf_floats = 3 * kStage * DP + kStage * cols + 8 * kStage;
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const int hk = h / (heads / kv_heads);
    const int q0 = q_start[blockIdx.z], q1 = q_start[blockIdx.z + 1];
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int block_col0 = blockIdx.x * cols;
    const int col0 = block_col0 + warp * WC;
    float* st = state + (size_t)slots[blockIdx.z] * state_stride + (size_t)h * dv * d;
    constexpr int RQ = 2 * DP + 4, RG = DP + 4;
    const bool v16 = (dv & 3) == 0 && (cols & 3) == 0 && (((uintptr_t)vin) & 15) == 0;          // the values' rows in pieces of 16 bytes
    auto stage = [&](int b, int t0) {
        float* qs = smem + (size_t)b * buf_floats;
        float* ks = qs + kStage * DP;
        float* as = ks + kStage * DP;
        float* vs = as + kStage * DP;
        float* sb = vs + kStage * cols;
        float* sq = sb + 4 * kStage;
        const int nt = min(kStage, q1 - t0);
        for (int idx = threadIdx.x; idx < nt * (DP / 4); idx += blockDim.x) {
            const int tk = idx / (DP / 4), i = idx - tk * (DP / 4);
            const float* rq = prep_qk + ((size_t)(t0 + tk) * kv_heads + hk) * RQ;
            const float* rg = prep_g + ((size_t)(t0 + tk) * heads + h) * RG;
            stage16(qs + tk * DP + 4 * i, rq + 4 * i, true);
            stage16(ks + tk * DP + 4 * i, rq + DP + 4 * i, true);
            stage16(as + tk * DP + 4 * i, rg + 4 * i, true);
        }
        for (int tk = threadIdx.x; tk < nt; tk += blockDim.x) {
            stage16(sb + 4 * tk, prep_g + ((size_t)(t0 + tk) * heads + h) * RG + DP, true);
            stage16(sq + 4 * tk, prep_qk + ((size_t)(t0 + tk) * kv_heads + hk) * RQ + 2 * DP, true);
        }
        if (v16) {
            for (int e = threadIdx.x; e < nt * (cols / 4); e += blockDim.x) {
                const int tk = e / (cols / 4), j4 = e - tk * (cols / 4);
                const int c = block_col0 + 4 * j4;
                stage16(vs + tk * cols + 4 * j4, vin + (size_t)(t0 + tk) * heads * dv + h * dv + (c < dv ? c : 0), c < dv);
            }
        } else {
            for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
                const int tk = e / cols, j = e - tk * cols;
                const int c = block_col0 + j;
                vs[e] = c < dv ? vin[(size_t)(t0 + tk) * heads * dv + h * dv + c] : 0.0f;
            }
        }
        asm volatile("cp.async.commit_group;");
    };
    stage(0, q0);
    float S[WC][E];
#pragma unroll
    for (int j = 0; j < WC; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e) S[j][e] = (col0 + j < dv && E * lane + e < d) ? st[(size_t)(col0 + j) * d + E * lane + e] : 0.0f;
    int b = 0;
    for (int t0 = q0; t0 < q1; t0 += kStage, b ^= 1) {
        const int nt = min(kStage, q1 - t0);
        asm volatile("cp.async.wait_group 0;");
        __syncthreads();                     // this stage has landed for everybody, and everybody has left the other buffer
        if (t0 + kStage < q1) stage(b ^ 1, t0 + kStage);
        const float* qs = smem + (size_t)b * buf_floats;
        const float* ks = qs + kStage * DP;
        const float* as = ks + kStage * DP;
        const float* vs = as + kStage * DP;
        const float* sb = vs + kStage * cols;
        const float* sq = sb + 4 * kStage;
#pragma unroll 2
        for (int tk = 0; tk < nt; ++tk) {
            float kk[E], aa[E], qq[E], v[WC], acck[WC], accq[WC];
            load_elements<E>(kk, ks + tk * DP + E * lane);
            load_elements<E>(aa, as + tk * DP + E * lane);
            load_elements<E>(qq, qs + tk * DP + E * lane);
            load_elements<WC>(v, vs + tk * cols + warp * WC);
            const float beta = sb[4 * tk], kq = sq[4 * tk];
#pragma unroll
            for (int j = 0; j < WC; ++j) {
                acck[j] = accq[j] = 0.0f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    S[j][e] *= aa[e];
                    acck[j] = fmaf(S[j][e], kk[e], acck[j]);
                    accq[j] = fmaf(S[j][e], qq[e], accq[j]);
                }
            }
            const float sk = sum_across_warp<WC>(acck, lane), sqv = sum_across_warp<WC>(accq, lane);
            const int jm = column_after_sum<WC>(lane);                   // the column whose sums this lane holds now
            float vm = v[0];
#pragma unroll
            for (int j = 1; j < WC; ++j) vm = jm == j ? v[j] : vm;
            const float um = beta * (vm - sk);
            if (sum_is_first<WC>(lane) && col0 + jm < dv) out[(size_t)(t0 + tk) * heads * dv + h * dv + col0 + jm] = fmaf(um, kq, sqv);
#pragma unroll
            for (int j = 0; j < WC; ++j) {
                const float u = __shfl_sync(0xffffffffu, um, lane_of_column<WC>(j));
#pragma unroll
                for (int e = 0; e < E; ++e) S[j][e] = fmaf(kk[e], u, S[j][e]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < WC; ++j)
#pragma unroll
        for (int e = 0; e < E; ++e)
            if (col0 + j < dv && E * lane + e < d) st[(size_t)(col0 + j) * d + E * lane + e] = S[j][e];
}

// The selective scan with a state row per channel.  x [T, x_stride] at column x_off (after its convolution and activation),
// bc [T, bc_stride]: B at column b_off, C at c_off (N each, shared by all channels), dt_raw [T, dt_stride] float (before the
// softplus), z [T, z_stride] at z_off: the gate.  A channel is a column of the walk: a warp holds eight channels, each lane
// E neighbouring state elements of all eight, and the channels' rates -exp(A_log) log2(e), so that a decay is one exp2.
// The chunk's decay of channel c and element n is exp2(rate[c, n] * the sum of the chunk's step sizes of c).
template <typename T, int E>
__global__ void __launch_bounds__(512)
channel_scan_kernel(const T* __restrict__ x, int x_stride, int x_off, const T* __restrict__ bc, int bc_stride, int b_off, int c_off,
                    const float* __restrict__ dt_raw, int dt_stride, const T* __restrict__ z, int z_stride, int z_off,
                    const float* __restrict__ A_log, const float* __restrict__ D, float* __restrict__ state, long long state_stride,
                    const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ y, int inner, int N,
                    const int* __restrict__ seg, int mode, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    constexpr int NP = 32 * E;
    const int warps = blockDim.x >> 5, cols = kWarpCols * warps;
    extern __shared__ __align__(16) float smem[];
    float* Bs = smem;                           // [kStage][NP]
    float* Cs = Bs + kStage * NP;               // [kStage][NP]
    float* xs = Cs + kStage * NP;               // [kStage][cols]
    float* dts = xs + kStage * cols;            // [kStage][cols] step sizes
    pdl_launch_dependents();
    pdl_wait();
    const Piece pc = piece_of(seg, q_start, slots);
    const int q0 = pc.q0, q1 = pc.q1;
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * cols + warp * kWarpCols;          // this warp's first channel
    float* st = state + (size_t)pc.slot * state_stride;
    float* cst = chunk_state ? chunk_state + (size_t)pc.chunk * inner * N : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[kWarpCols][E], rate[kWarpCols][E], dtsum[kWarpCols];
#pragma unroll
    for (int j = 0; j < kWarpCols; ++j) {
        dtsum[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const bool in = col0 + j < inner && E * lane + e < N;
            const size_t at = (size_t)(col0 + j) * N + E * lane + e;
            S[j][e] = (mode != kScanLocal && in) ? from[at] : 0.0f;
            rate[j][e] = in ? -expf(A_log[at]) * 1.4426950408889634f : 0.0f;
        }
    }
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();                                   // the stage before has been used up
        for (int tk = warp; tk < nt; tk += warps) {
            const T* row = bc + (size_t)(t0 + tk) * bc_stride;
            for (int n = lane; n < NP; n += 32) {
                Bs[tk * NP + n] = n < N ? to_float(row[b_off + n]) : 0.0f;
                if (mode != kScanLocal) Cs[tk * NP + n] = n < N ? to_float(row[c_off + n]) : 0.0f;
            }
        }
        for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
            const int tk = e / cols, j = e - tk * cols;
            const int c = blockIdx.x * cols + j;
            xs[e] = c < inner ? to_float(x[(size_t)(t0 + tk) * x_stride + x_off + c]) : 0.0f;
            dts[e] = c < inner ? softplus_f(dt_raw[(size_t)(t0 + tk) * dt_stride + c]) : 0.0f;
        }
        __syncthreads();
#pragma unroll 2
        for (int tk = 0; tk < nt; ++tk) {
            float b[E], xv[kWarpCols], dt[kWarpCols];
            load_elements<E>(b, Bs + tk * NP + E * lane);
            load_elements<kWarpCols>(xv, xs + tk * cols + warp * kWarpCols);
            load_elements<kWarpCols>(dt, dts + tk * cols + warp * kWarpCols);
            if (mode == kScanLocal) {
#pragma unroll
                for (int j = 0; j < kWarpCols; ++j) {
                    const float dx = dt[j] * xv[j];
                    dtsum[j] += dt[j];
#pragma unroll
                    for (int e = 0; e < E; ++e) S[j][e] = fmaf(exp2f(dt[j] * rate[j][e]), S[j][e], b[e] * dx);
                }
                continue;
            }
            float cc[E], acc[kWarpCols];
            load_elements<E>(cc, Cs + tk * NP + E * lane);
#pragma unroll
            for (int j = 0; j < kWarpCols; ++j) {
                const float dx = dt[j] * xv[j];
                acc[j] = 0.0f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    S[j][e] = fmaf(exp2f(dt[j] * rate[j][e]), S[j][e], b[e] * dx);
                    acc[j] = fmaf(S[j][e], cc[e], acc[j]);
                }
            }
            const float total = sum8_across_warp(acc, lane);
            const int j = column_after_sum8(lane);
            if ((lane & 3) == 0 && col0 + j < inner) {
                const int c = col0 + j;
                const float r = fmaf(D[c], xs[tk * cols + warp * kWarpCols + j], total);
                y[(size_t)(t0 + tk) * inner + c] = from_float<T>(r * silu_f(to_float(z[(size_t)(t0 + tk) * z_stride + z_off + c])));
            }
        }
    }
    if (mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int j = 0; j < kWarpCols; ++j)
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (col0 + j < inner && E * lane + e < N) {
                    const size_t at = (size_t)(col0 + j) * N + E * lane + e;
                    to[at] = S[j][e];
                    if (mode == kScanLocal) chunk_decay[(size_t)pc.chunk * inner * N + at] = exp2f(dtsum[j] * rate[j][e]);
                }
    }
}

// The same scan for states of up to 64 elements, a channel per thread: the channel's whole state row and its rates stay in
// the thread's registers (NB of each, N <= NB, the rest zeros that stay zeros), so the sum over the state is a chain of
// multiply-adds inside the thread and nothing crosses lanes.  With a state of 16 the form above leaves half of every warp
// idle and pays nine shuffles a token for eight short sums.  B and C of kStage tokens are staged once a block (every thread
// reads the same address: one 16-byte load serves the warp); step sizes, inputs and gates are staged by the thread that
// uses them, with softplus and silu applied.  A token's decays are ex2.approx of a product that is never positive (a result
// below the smallest normal float is zero).  Same arguments, passes and state layout as channel_scan_kernel.
constexpr int kLaneChannels = 128;      // threads of a block, a channel each

template <typename T, int NB>
__global__ void __launch_bounds__(kLaneChannels)
channel_scan_lane_kernel(const T* __restrict__ x, int x_stride, int x_off, const T* __restrict__ bc, int bc_stride, int b_off, int c_off,
                         const float* __restrict__ dt_raw, int dt_stride, const T* __restrict__ z, int z_stride, int z_off,
                         const float* __restrict__ A_log, const float* __restrict__ D, float* __restrict__ state, long long state_stride,
                         const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ y, int inner, int N,
                         const int* __restrict__ seg, int mode, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    __shared__ __align__(16) float Bs[kStage][NB];
    __shared__ __align__(16) float Cs[kStage][NB];
    __shared__ float xs[kStage][kLaneChannels];
    __shared__ float dts[kStage][kLaneChannels];
    __shared__ float gs[kStage][kLaneChannels];         // silu of the gate
    pdl_launch_dependents();
    pdl_wait();
    const Piece pc = piece_of(seg, q_start, slots);
    const int q0 = pc.q0, q1 = pc.q1;
    if (q1 <= q0) return;
    const int tid = threadIdx.x;
    const int c = blockIdx.x * kLaneChannels + tid;
    const bool live = c < inner;
    float* st = state + (size_t)pc.slot * state_stride;
    float* cst = chunk_state ? chunk_state + (size_t)pc.chunk * inner * N : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[NB], rate[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        const bool in = live && n < N;
        const size_t at = (size_t)c * N + n;
        S[n] = (mode != kScanLocal && in) ? from[at] : 0.0f;
        rate[n] = in ? -expf(A_log[at]) * 1.4426950408889634f : 0.0f;
    }
    const float dc = live ? D[c] : 0.0f;
    float dtsum = 0.0f;
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();                                   // the stage before has been used up
        for (int e = tid; e < nt * NB; e += kLaneChannels) {
            const int tk = e / NB, n = e - tk * NB;
            const T* row = bc + (size_t)(t0 + tk) * bc_stride;
            Bs[tk][n] = n < N ? to_float(row[b_off + n]) : 0.0f;
            if (mode != kScanLocal) Cs[tk][n] = n < N ? to_float(row[c_off + n]) : 0.0f;
        }
        if (live) {
#pragma unroll 8
            for (int tk = 0; tk < nt; ++tk) {
                xs[tk][tid] = to_float(x[(size_t)(t0 + tk) * x_stride + x_off + c]);
                dts[tk][tid] = softplus_f(dt_raw[(size_t)(t0 + tk) * dt_stride + c]);
                if (mode != kScanLocal) gs[tk][tid] = silu_f(to_float(z[(size_t)(t0 + tk) * z_stride + z_off + c]));
            }
        }
        __syncthreads();
        if (!live) continue;
        for (int tk = 0; tk < nt; ++tk) {
            const float dt = dts[tk][tid], xv = xs[tk][tid], dx = dt * xv;
            if (mode == kScanLocal) {
                dtsum += dt;
#pragma unroll
                for (int n = 0; n < NB; n += 4) {
                    const float4 b = *reinterpret_cast<const float4*>(&Bs[tk][n]);
                    S[n] = fmaf(fast_exp2(dt * rate[n]), S[n], b.x * dx);
                    S[n + 1] = fmaf(fast_exp2(dt * rate[n + 1]), S[n + 1], b.y * dx);
                    S[n + 2] = fmaf(fast_exp2(dt * rate[n + 2]), S[n + 2], b.z * dx);
                    S[n + 3] = fmaf(fast_exp2(dt * rate[n + 3]), S[n + 3], b.w * dx);
                }
                continue;
            }
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;       // four sums side by side, always added in the same order
#pragma unroll
            for (int n = 0; n < NB; n += 4) {
                const float4 b = *reinterpret_cast<const float4*>(&Bs[tk][n]);
                const float4 cc = *reinterpret_cast<const float4*>(&Cs[tk][n]);
                S[n] = fmaf(fast_exp2(dt * rate[n]), S[n], b.x * dx);
                S[n + 1] = fmaf(fast_exp2(dt * rate[n + 1]), S[n + 1], b.y * dx);
                S[n + 2] = fmaf(fast_exp2(dt * rate[n + 2]), S[n + 2], b.z * dx);
                S[n + 3] = fmaf(fast_exp2(dt * rate[n + 3]), S[n + 3], b.w * dx);
                a0 = fmaf(S[n], cc.x, a0);
                a1 = fmaf(S[n + 1], cc.y, a1);
                a2 = fmaf(S[n + 2], cc.z, a2);
                a3 = fmaf(S[n + 3], cc.w, a3);
            }
            const float r = fmaf(dc, xv, (a0 + a1) + (a2 + a3));
            y[(size_t)(t0 + tk) * inner + c] = from_float<T>(r * gs[tk][tid]);
        }
    }
    if (mode != kScanApply && live) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int n = 0; n < NB; ++n)
            if (n < N) {
                const size_t at = (size_t)c * N + n;
                to[at] = S[n];
                if (mode == kScanLocal) chunk_decay[(size_t)pc.chunk * inner * N + at] = exp2f(dtsum * rate[n]);
            }
    }
}

// Between the two passes over chunks: for each run of chunks (a sequence's, in order) S starts as the slot's state;
// chunk_state[chunk] (the chunk's end state from zeros) is replaced by the state the chunk starts from, and
// S <- decay[chunk, head] S + end state.  The last S goes back to the slot.
__global__ void scan_carry_kernel(float* __restrict__ state, long long state_stride, float* __restrict__ chunk_state,
                                  const float* __restrict__ chunk_decay, const float* __restrict__ token_decay, const int* __restrict__ seg,
                                  const int* __restrict__ runs, int heads, int per_head, int period) {
    pdl_launch_dependents();
    pdl_wait();
    const int first = runs[3 * blockIdx.y], count = runs[3 * blockIdx.y + 1], slot = runs[3 * blockIdx.y + 2];
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int elements = heads * per_head;
    if (e >= elements) return;
    const int h = e / per_head;
    // a decay per chunk and head (period 0), or `period` of them per head: element i of a head takes number i % period
    const int per_chunk = period > 0 ? heads * period : heads;
    const int dec_at = period > 0 ? h * period + (e - h * per_head) % period : h;
    float* st = state + (size_t)slot * state_stride + e;
    float S = *st;
    for (int c0 = first; c0 < first + count; c0 += 8) {
        // eight chunks' end states and decays are asked for at once: they do not depend on S
        float z[8], dec[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + u;
            const bool in = c < first + count;
            z[u] = in ? chunk_state[(size_t)c * elements + e] : 0.0f;
            // the chunk's decay: given, or a constant per token and head to the power of the chunk's length
            dec[u] = !in ? 1.0f : chunk_decay ? chunk_decay[(size_t)c * per_chunk + dec_at] : powf(token_decay[h], (float)(seg[4 * c + 1] - seg[4 * c]));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < first + count) {
                chunk_state[(size_t)(c0 + u) * elements + e] = S;
                S = fmaf(dec[u], S, z[u]);
            }
        }
    }
    *st = S;
}

// One block per (token, group).  mode 0: v = y silu(z), out = v rinv w; mode 1: out = y rinv w sigmoid(z); mode 2: out = y rinv w silu(z).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, int gate_off, const float* __restrict__ w,
                                     float eps, int mode, T* __restrict__ out, int n, int groups) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups;
    const int gs = n / groups;
    const float* yr = y + (size_t)t * n + (size_t)g * gs;
    const T* zr = gate + (size_t)t * gate_stride + gate_off + (size_t)g * gs;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < gs; j += blockDim.x) {
        float v = yr[j];
        if (mode == 0) v *= silu_f(to_float(zr[j]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)gs + eps);
    T* o = out + (size_t)t * n + (size_t)g * gs;
    for (int j = threadIdx.x; j < gs; j += blockDim.x) {
        float v = yr[j];
        const float z = to_float(zr[j]);
        if (mode == 0) v = (v * silu_f(z)) * rinv * w[g * gs + j];
        else if (mode == 1) v = (v * rinv * w[g * gs + j]) * sigmoid_f(z);
        else v = (v * rinv * w[g * gs + j]) * silu_f(z);
        o[j] = from_float<T>(v);
    }
}

// The same for groups of up to kWarpGroup elements (a head's output): a warp per (token, group), eight of them a block, no
// barrier; a lane keeps its elements (with the gate applied where it comes first) between the sum and the result.
constexpr int kWarpGroup = 512;

template <typename T, bool kVec4>
__global__ void __launch_bounds__(256)
gated_rmsnorm_warp_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, int gate_off, const float* __restrict__ w,
                          float eps, int mode, T* __restrict__ out, int n, int groups, long long rows) {
    pdl_launch_dependents();
    pdl_wait();
    const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = r / groups;
    const int g = (int)(r - t * groups);
    const int gs = n / groups;
    const float* yr = y + (size_t)t * n + (size_t)g * gs;
    const T* zr = gate + (size_t)t * gate_stride + gate_off + (size_t)g * gs;
    const float* wr = w + (size_t)g * gs;
    T* o = out + (size_t)t * n + (size_t)g * gs;
    constexpr int kPer = kWarpGroup / 32;
    float v[kPer], zz[kPer];
    float ss = 0.0f;
    // kVec4 (every row and group starts at a multiple of four elements): a lane takes four neighbouring elements at a time
    // with one load each of y and of the gate; otherwise one element at a time, a warp's 32 side by side
    constexpr int kStep = kVec4 ? 4 : 1;
#pragma unroll
    for (int i = 0; i < kPer; i += kStep) {
        const int j = kVec4 ? 4 * lane + 32 * i : lane + 32 * i;
        if constexpr (kVec4) {
            if (j < gs) {
                const float4 a = *reinterpret_cast<const float4*>(yr + j);
                v[i] = a.x; v[i + 1] = a.y; v[i + 2] = a.z; v[i + 3] = a.w;
                if constexpr (sizeof(T) == 2) {
                    const uint2 b = *reinterpret_cast<const uint2*>(zr + j);
                    zz[i] = __uint_as_float(b.x << 16); zz[i + 1] = __uint_as_float(b.x & 0xffff0000u);
                    zz[i + 2] = __uint_as_float(b.y << 16); zz[i + 3] = __uint_as_float(b.y & 0xffff0000u);
                } else {
                    const float4 b = *reinterpret_cast<const float4*>(zr + j);
                    zz[i] = b.x; zz[i + 1] = b.y; zz[i + 2] = b.z; zz[i + 3] = b.w;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) v[i + q] = zz[i + q] = 0.0f;
            }
        } else {
            v[i] = j < gs ? yr[j] : 0.0f;
            zz[i] = j < gs ? to_float(zr[j]) : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < kStep; ++q) {
            if (mode == 0) v[i + q] *= silu_f(zz[i + q]);
            ss += v[i + q] * v[i + q];
        }
    }
    ss = warp_sum(ss);
    const float rinv = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int i = 0; i < kPer; i += kStep) {
        const int j = kVec4 ? 4 * lane + 32 * i : lane + 32 * i;
        if (j >= gs) break;
        float u[kStep];
#pragma unroll
        for (int q = 0; q < kStep; ++q) {
            u[q] = v[i + q] * rinv * wr[j + q];
            if (mode == 1) u[q] *= sigmoid_f(zz[i + q]);
            else if (mode == 2) u[q] *= silu_f(zz[i + q]);
        }
        if constexpr (kVec4) {
            if constexpr (sizeof(T) == 2) {
                __nv_bfloat162 pk[2] = {__floats2bfloat162_rn(u[0], u[1]), __floats2bfloat162_rn(u[2], u[3])};
                *reinterpret_cast<uint2*>(o + j) = *reinterpret_cast<const uint2*>(pk);
            } else {
                *reinterpret_cast<float4*>(o + j) = make_float4(u[0], u[1], u[2], u[3]);
            }
        } else {
            o[j] = from_float<T>(u[0]);
        }
    }
}

}  // namespace

// shift: every sequence of the step has one token (the caller's promise), and the state moves on in the same launch.
LI_EXPORT int li_causal_conv_silu(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* b, float* state,
                                  long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
                                  void* out, int T, int C, int taps, int shift, cudaStream_t stream) {
    LI_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal convolution: %d taps (1..%d)", taps, kMaxTaps);
    LI_REQUIRE(C > 0 && in_off >= 0 && in_off + C <= in_stride, "causal convolution: %d channels at column %d of %d", C, in_off, in_stride);
    if (T == 0) return 0;
    LI_REQUIRE(T <= 65535, "causal convolution: %d tokens in one launch", T);
    const dim3 grid(ceil_div(C, 128), T);
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(causal_conv_silu_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, in_stride, in_off, w, b, state, state_stride,
                          state_off, q_start, seq_of_token, slots, (float*)out, C, taps, shift);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(causal_conv_silu_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, in_stride, in_off, w, b, state, state_stride,
                          state_off, q_start, seq_of_token, slots, (bf16*)out, C, taps, shift);
    else
        return li_fail("causal convolution: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("causal convolution: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("causal_conv_silu");
}

LI_EXPORT int li_conv_state_shift(const void* in, int dtype, int in_stride, int in_off, float* state, long long state_stride, long long state_off,
                                  const int* q_start, const int* slots, int S, int C, int taps, cudaStream_t stream) {
    LI_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal convolution: %d taps (1..%d)", taps, kMaxTaps);
    if (S == 0 || taps == 1) return 0;
    LI_REQUIRE(S <= 65535, "causal convolution: %d sequences in one launch", S);
    const dim3 grid(ceil_div(C, 128), S);
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(conv_state_shift_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, in_stride, in_off, state, state_stride, state_off,
                          q_start, slots, C, taps);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(conv_state_shift_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, in_stride, in_off, state, state_stride, state_off,
                          q_start, slots, C, taps);
    else
        return li_fail("causal convolution: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("conv_state_shift: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("conv_state_shift");
}

// warps of a block: enough for the head's columns, at most 16
static int scan_warps(int columns) {
    const int w = ceil_div(columns, kWarpCols);
    return w >= 16 ? 16 : w >= 8 ? 8 : w >= 4 ? 4 : w >= 2 ? 2 : 1;
}

template <typename T, int E>
static int launch_ssm(const void* xbc, int C, const void* dt_raw, int dt_stride, const float* dt_bias, const float* A_log, const float* D,
                      float* state, long long state_stride, const int* q_start, const int* slots, float* y, int S, int heads, int P, int N,
                      int groups, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    const int warps = scan_warps(P), cols = warps * kWarpCols;
    const size_t smem = ((size_t)2 * kStage * 32 * E + kStage * cols + 2 * kStage) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(ssm_scan_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(ssm_scan_kernel<T, E>, dim3(ceil_div(P, cols), heads, S), dim3(warps * 32), smem, stream, (const T*)xbc, C,
                                  (const T*)dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, heads, P, N, groups, seg, mode,
                                  chunk_state, chunk_decay);
    if (e != cudaSuccess) return li_fail("ssm_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("ssm_scan");
}

// The state of a slot: [heads][P][N] (a column of the head's N x P matrix at a time).
LI_EXPORT int li_ssm_scan(const void* xbc, int dtype, int C, const void* dt_raw, int dt_stride, const float* dt_bias, const float* A_log,
                          const float* D, float* state, long long state_stride, const int* q_start, const int* slots, float* y, int S, int heads,
                          int P, int N, int groups, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && chunk_decay != nullptr && (uintptr_t)seg % 16 == 0),
               "state-space scan: pass %d needs the chunks, their states and their decays (or none of them)", mode);
    LI_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "state-space scan: %d heads in %d groups", heads, groups);
    LI_REQUIRE(P > 0 && N > 0 && N <= 256, "state-space scan: head size %d, state size %d (at most 256)", P, N);
    LI_REQUIRE(C == heads * P + 2 * groups * N, "state-space scan: %d channels for %d heads of %d and %d groups of %d", C, heads, P, groups, N);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "state-space scan: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "state-space scan: %d sequences or %d heads in one launch", S, heads);
#define LI_SCAN(RR)                                                                                                                            \
    return dtype == LI_F32 ? launch_ssm<float, RR>(xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, S, heads, \
                                                   P, N, groups, seg, mode, chunk_state, chunk_decay, stream)                                  \
                           : launch_ssm<bf16, RR>(xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, S, heads,  \
                                                  P, N, groups, seg, mode, chunk_state, chunk_decay, stream)
    if (N <= 32) { LI_SCAN(1); }
    if (N <= 64) { LI_SCAN(2); }
    if (N <= 128) { LI_SCAN(4); }
    LI_SCAN(8);
#undef LI_SCAN
}

template <typename T, int E>
static int launch_decay(const void* qkv, int stride, int q_off, int k_off, int v_off, const float* decay, float* state, long long state_stride,
                        const int* q_start, const int* slots, float* out, int S, int heads, int d, int dv, const int* seg, int mode,
                        float* chunk_state, cudaStream_t stream) {
    const int warps = scan_warps(dv), cols = warps * kWarpCols;
    const size_t smem = ((size_t)2 * kStage * 32 * E + kStage * cols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(decay_scan_kernel<T, E>, dim3(ceil_div(dv, cols), heads, S), dim3(warps * 32), smem, stream, (const T*)qkv, stride,
                                  q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, heads, d, dv, seg, mode, chunk_state);
    if (e != cudaSuccess) return li_fail("decay_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("decay_scan");
}

// The state of a slot: [heads][dv][d] (a column of the head's d x dv matrix at a time).
LI_EXPORT int li_decay_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* decay, float* state,
                            long long state_stride, const int* q_start, const int* slots, float* out, int S, int heads, int d, int dv,
                            const int* seg, int mode, float* chunk_state, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && (uintptr_t)seg % 16 == 0),
               "decay scan: pass %d needs the chunks and their states (or none of them)", mode);
    LI_REQUIRE(heads > 0 && d > 0 && d <= 256 && dv > 0, "decay scan: %d heads of %d x %d (keys of at most 256)", heads, d, dv);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "decay scan: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "decay scan: %d sequences or %d heads in one launch", S, heads);
#define LI_SCAN(RR)                                                                                                                          \
    return dtype == LI_F32 ? launch_decay<float, RR>(qkv, stride, q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, S, heads, \
                                                     d, dv, seg, mode, chunk_state, stream)                                                  \
                           : launch_decay<bf16, RR>(qkv, stride, q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, S, heads,  \
                                                    d, dv, seg, mode, chunk_state, stream)
    if (d <= 32) { LI_SCAN(1); }
    if (d <= 64) { LI_SCAN(2); }
    if (d <= 128) { LI_SCAN(4); }
    LI_SCAN(8);
#undef LI_SCAN
}

template <typename T, int E>
static int launch_gla(const void* qkv, int stride, int q_off, int k_off, int v_off, const float* za, int za_stride, int za_off, float inv_tau,
                      float q_scale, float* state, long long state_stride, const int* q_start, const int* slots, float* out, int S, int heads,
                      int d, int dv, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    const int warps = scan_warps(dv), cols = warps * kWarpCols;
    const size_t smem = ((size_t)3 * kStage * 32 * E + kStage * cols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gla_scan_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(gla_scan_kernel<T, E>, dim3(ceil_div(dv, cols), heads, S), dim3(warps * 32), smem, stream, (const T*)qkv, stride,
                                  q_off, k_off, v_off, za, za_stride, za_off, inv_tau, q_scale, state, state_stride, q_start, slots, out, heads, d, dv,
                                  seg, mode, chunk_state, chunk_decay);
    if (e != cudaSuccess) return li_fail("gla_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("gla_scan");
}

// The state of a slot: [heads][dv][d] (a column of the head's d x dv matrix at a time).  chunk_decay: [chunks, heads, d].
LI_EXPORT int li_gla_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* za, int za_stride, int za_off,
                          float inv_tau, float q_scale, float* state, long long state_stride, const int* q_start, const int* slots, float* out,
                          int S, int heads, int d, int dv, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && chunk_decay != nullptr && (uintptr_t)seg % 16 == 0),
               "gated linear attention: pass %d needs the chunks, their states and their decays (or none of them)", mode);
    LI_REQUIRE(heads > 0 && d > 0 && d <= 256 && dv > 0, "gated linear attention: %d heads of %d x %d (keys of at most 256)", heads, d, dv);
    LI_REQUIRE(za != nullptr && za_off >= 0 && za_off + heads * d <= za_stride, "gated linear attention: decays at column %d of %d", za_off, za_stride);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "gated linear attention: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "gated linear attention: %d sequences or %d heads in one launch", S, heads);
#define LI_SCAN(RR)                                                                                                                              \
    return dtype == LI_F32 ? launch_gla<float, RR>(qkv, stride, q_off, k_off, v_off, za, za_stride, za_off, inv_tau, q_scale, state, state_stride,  \
                                                   q_start, slots, out, S, heads, d, dv, seg, mode, chunk_state, chunk_decay, stream)           \
                           : launch_gla<bf16, RR>(qkv, stride, q_off, k_off, v_off, za, za_stride, za_off, inv_tau, q_scale, state, state_stride,   \
                                                  q_start, slots, out, S, heads, d, dv, seg, mode, chunk_state, chunk_decay, stream)
    if (d <= 32) { LI_SCAN(1); }
    if (d <= 64) { LI_SCAN(2); }
    if (d <= 128) { LI_SCAN(4); }
    LI_SCAN(8);
#undef LI_SCAN
}

// key channels a lane holds for keys of d elements (rows of the prepared vectors have 32 E floats)
static int delta_elements(int d) { return d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8; }
constexpr int kDeltaWarps = 4;          // warps of a block of the walk at most
static int g_delta_cols = 0;            // 0: columns a warp by the size of the launch; 2, 4 or 8: that many, for tests and measurements

template <int E, int WC>
static int launch_delta(const float* prep_qk, const float* prep_g, const float* v, float* state, long long state_stride, const int* q_start,
                        const int* slots, float* out, int S, int heads, int kv_heads, int d, int dv, cudaStream_t stream) {
    int warps = ceil_div(dv, WC);
    warps = warps >= kDeltaWarps ? kDeltaWarps : warps >= 2 ? 2 : 1;
    const int cols = warps * WC;
    const size_t smem = 2 * ((size_t)3 * kStage * 32 * E + kStage * cols + 8 * kStage) * sizeof(float);          // two buffers
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<E, WC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(delta_scan_kernel<E, WC>, dim3(ceil_div(dv, cols), heads, S), dim3(warps * 32), smem, stream, prep_qk, prep_g, v, state,
                                  state_stride, q_start, slots, out, heads, kv_heads, d, dv);
    if (e != cudaSuccess) return li_fail("delta_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("delta_scan");
}

// Columns a warp: four while that leaves the launch under about two warps a scheduler (148 multiprocessors of four), else eight.
// Measured at 2,048 tokens of one sequence, 12 heads of 128 x 128: 0.69 ms with eight, 0.54 with four, 0.57 with two (kept for
// measurements).  The result does not depend on it (sum_across_warp).
static int delta_cols(int S, int heads, int dv) {
    if (g_delta_cols) return g_delta_cols;
    const long long columns = (long long)S * heads * dv;
    return columns / 8 >= 1184 ? 8 : 4;
}

template <int E>
static int launch_delta_cols(const float* prep_qk, const float* prep_g, const float* v, float* state, long long state_stride, const int* q_start,
                             const int* slots, float* out, int S, int heads, int kv_heads, int d, int dv, cudaStream_t stream) {
    switch (delta_cols(S, heads, dv)) {
        case 8: return launch_delta<E, 8>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
        case 4: return launch_delta<E, 4>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
        default: return launch_delta<E, 2>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
    }
}

// What the walk of the gated delta rule needs of every token, from the projections (see delta_prepare_kernel).  proj [T, stride]
// holds the convolution's channels q | k | v (kv_heads d, kv_heads d, heads dv) from column col0 and beta's input at b_off + h;
// conv_w [channels, taps]; the state holds the last taps - 1 inputs at state_off ([taps - 1, channels], oldest first);
// za [T, za_stride] float: the decays' input at za_off + h d + i.  Outputs: prep_qk [T, kv_heads, 2 DP + 4], prep_g
// [T, heads, DP + 4], v [T, heads dv], float, with DP = 32, 64, 128 or 256 (the first that holds d).
LI_EXPORT int li_delta_prepare(const void* proj, int dtype, int stride, int col0, int b_off, const float* conv_w, int taps, float* state,
                               long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
                               const float* za, int za_stride, int za_off, const float* A_log, float q_scale, float unit_eps, float* prep_qk,
                               float* prep_g, float* v, int T, int heads, int kv_heads, int d, int dv, int shift, cudaStream_t stream) {
    LI_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && d > 0 && d <= 256 && dv > 0,
               "delta rule: %d heads on %d key heads of %d x %d (keys of at most 256)", heads, kv_heads, d, dv);
    LI_REQUIRE(taps >= 1 && taps <= kMaxTaps && conv_w != nullptr, "delta rule: a convolution of %d taps (at most %d)", taps, kMaxTaps);
    LI_REQUIRE(za != nullptr && za_off >= 0 && za_off + heads * d <= za_stride, "delta rule: decays at column %d of %d", za_off, za_stride);
    LI_REQUIRE(col0 >= 0 && col0 + 2 * kv_heads * d + heads * dv <= stride && b_off >= 0 && b_off + heads <= stride && A_log != nullptr,
               "delta rule: the projections' columns do not fit rows of %d", stride);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "delta rule: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const int DP = 32 * delta_elements(d);
    const long long warps = (long long)T * (kv_heads + 2 * heads);
    const dim3 grid((unsigned)ceil_div_ll(warps, 4));
    cudaError_t e;
#define LI_PREPARE(TT, TAPS_)                                                                                                                  \
    e = li_launch_pdl(delta_prepare_kernel<TT, TAPS_>, grid, dim3(128), 0, stream, (const TT*)proj, stride, col0, b_off, conv_w, taps, state,     \
                      state_stride, state_off, q_start, seq_of_token, slots, za, za_stride, za_off, A_log, q_scale, unit_eps, prep_qk, prep_g, v, T, \
                      heads, kv_heads, d, dv, DP, shift)
    if (dtype == LI_F32) {
        if (taps == 4) LI_PREPARE(float, 4);
        else if (taps == 3) LI_PREPARE(float, 3);
        else if (taps == 2) LI_PREPARE(float, 2);
        else LI_PREPARE(float, 0);
    } else {
        if (taps == 4) LI_PREPARE(bf16, 4);
        else if (taps == 3) LI_PREPARE(bf16, 3);
        else if (taps == 2) LI_PREPARE(bf16, 2);
        else LI_PREPARE(bf16, 0);
    }
#undef LI_PREPARE
    if (e != cudaSuccess) return li_fail("delta_prepare: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("delta_prepare");
}

// 0: columns a warp of the walk by the size of the launch; 2, 4 or 8: that many.  For tests and measurements.
LI_EXPORT void li_delta_force_columns(int columns) { g_delta_cols = (columns == 2 || columns == 4 || columns == 8) ? columns : 0; }

// The walk over what li_delta_prepare made.  The state of a slot: [heads][dv][d] (a column of the head's d x dv matrix at a time).
LI_EXPORT int li_delta_scan(const float* prep_qk, const float* prep_g, const float* v, float* state, long long state_stride, const int* q_start,
                            const int* slots, float* out, int S, int heads, int kv_heads, int d, int dv, cudaStream_t stream) {
    LI_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && d > 0 && d <= 256 && dv > 0,
               "delta rule: %d heads on %d key heads of %d x %d (keys of at most 256)", heads, kv_heads, d, dv);
    LI_REQUIRE(prep_qk != nullptr && prep_g != nullptr && v != nullptr && (uintptr_t)prep_qk % 16 == 0 && (uintptr_t)prep_g % 16 == 0,
               "delta rule: the prepared rows are missing or not on a 16-byte boundary");
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "delta rule: %d sequences or %d heads in one launch", S, heads);
    switch (delta_elements(d)) {
        case 1: return launch_delta_cols<1>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
        case 2: return launch_delta_cols<2>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
        case 4: return launch_delta_cols<4>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
        default: return launch_delta_cols<8>(prep_qk, prep_g, v, state, state_stride, q_start, slots, out, S, heads, kv_heads, d, dv, stream);
    }
}

template <typename T, int E>
static int launch_channel(const void* x, int x_stride, int x_off, const void* bc, int bc_stride, int b_off, int c_off, const float* dt_raw,
                          int dt_stride, const void* z, int z_stride, int z_off, const float* A_log, const float* D, float* state,
                          long long state_stride, const int* q_start, const int* slots, void* y, int S, int inner, int N, const int* seg, int mode,
                          float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    const int warps = scan_warps(inner) > 8 ? 8 : scan_warps(inner), cols = warps * kWarpCols;
    const size_t smem = ((size_t)2 * kStage * 32 * E + 2 * kStage * cols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(channel_scan_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(channel_scan_kernel<T, E>, dim3(ceil_div(inner, cols), 1, S), dim3(warps * 32), smem, stream, (const T*)x, x_stride,
                                  x_off, (const T*)bc, bc_stride, b_off, c_off, dt_raw, dt_stride, (const T*)z, z_stride, z_off, A_log, D, state,
                                  state_stride, q_start, slots, (T*)y, inner, N, seg, mode, chunk_state, chunk_decay);
    if (e != cudaSuccess) return li_fail("channel_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("channel_scan");
}

template <typename T, int NB>
static int launch_channel_lane(const void* x, int x_stride, int x_off, const void* bc, int bc_stride, int b_off, int c_off, const float* dt_raw,
                               int dt_stride, const void* z, int z_stride, int z_off, const float* A_log, const float* D, float* state,
                               long long state_stride, const int* q_start, const int* slots, void* y, int S, int inner, int N, const int* seg,
                               int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    cudaError_t e = li_launch_pdl(channel_scan_lane_kernel<T, NB>, dim3(ceil_div(inner, kLaneChannels), 1, S), dim3(kLaneChannels), 0, stream,
                                  (const T*)x, x_stride, x_off, (const T*)bc, bc_stride, b_off, c_off, dt_raw, dt_stride, (const T*)z, z_stride, z_off,
                                  A_log, D, state, state_stride, q_start, slots, (T*)y, inner, N, seg, mode, chunk_state, chunk_decay);
    if (e != cudaSuccess) return li_fail("channel_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("channel_scan");
}

// The state of a slot: [inner][N].  chunk_decay: [chunks, inner, N].
LI_EXPORT int li_channel_scan(const void* x, int dtype, int x_stride, int x_off, const void* bc, int bc_stride, int b_off, int c_off,
                              const float* dt_raw, int dt_stride, const void* z, int z_stride, int z_off, const float* A_log, const float* D,
                              float* state, long long state_stride, const int* q_start, const int* slots, void* y, int S, int inner, int N,
                              const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && chunk_decay != nullptr && (uintptr_t)seg % 16 == 0),
               "channel scan: pass %d needs the chunks, their states and their decays (or none of them)", mode);
    LI_REQUIRE(inner > 0 && N > 0 && N <= 256, "channel scan: %d channels with a state of %d (at most 256)", inner, N);
    LI_REQUIRE(x_off >= 0 && x_off + inner <= x_stride && z_off >= 0 && z_off + inner <= z_stride && inner <= dt_stride && b_off >= 0 &&
                   b_off + N <= bc_stride && c_off >= 0 && c_off + N <= bc_stride, "channel scan: columns outside their rows");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "channel scan: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535, "channel scan: %d sequences in one launch", S);
#define LI_SCAN(RR)                                                                                                                               \
    return dtype == LI_F32 ? launch_channel<float, RR>(x, x_stride, x_off, bc, bc_stride, b_off, c_off, dt_raw, dt_stride, z, z_stride, z_off, A_log, \
                                                       D, state, state_stride, q_start, slots, y, S, inner, N, seg, mode, chunk_state, chunk_decay, \
                                                       stream)                                                                                   \
                           : launch_channel<bf16, RR>(x, x_stride, x_off, bc, bc_stride, b_off, c_off, dt_raw, dt_stride, z, z_stride, z_off, A_log,  \
                                                      D, state, state_stride, q_start, slots, y, S, inner, N, seg, mode, chunk_state, chunk_decay,  \
                                                      stream)
#define LI_LANE(NB)                                                                                                                              \
    return dtype == LI_F32 ? launch_channel_lane<float, NB>(x, x_stride, x_off, bc, bc_stride, b_off, c_off, dt_raw, dt_stride, z, z_stride, z_off, \
                                                            A_log, D, state, state_stride, q_start, slots, y, S, inner, N, seg, mode, chunk_state, \
                                                            chunk_decay, stream)                                                                 \
                           : launch_channel_lane<bf16, NB>(x, x_stride, x_off, bc, bc_stride, b_off, c_off, dt_raw, dt_stride, z, z_stride, z_off,  \
                                                           A_log, D, state, state_stride, q_start, slots, y, S, inner, N, seg, mode, chunk_state,  \
                                                           chunk_decay, stream)
    // up to 64 state elements: a channel per thread, its row in registers; beyond: a warp per eight channels
    if (N <= 4) { LI_LANE(4); }
    if (N <= 8) { LI_LANE(8); }
    if (N <= 16) { LI_LANE(16); }
    if (N <= 32) { LI_LANE(32); }
    if (N <= 64) { LI_LANE(64); }
    if (N <= 128) { LI_SCAN(4); }
    LI_SCAN(8);
#undef LI_LANE
#undef LI_SCAN
}

// See scan_carry_kernel.  runs: triples (first chunk, chunks, slot); per_head: state elements of one head.  The decay of a
// chunk and head: chunk_decay[chunk, head], or (chunk_decay null) token_decay[head] to the power of the chunk's length; with
// period > 0 chunk_decay is [chunk, head, period] and element i of a head's state decays by number i % period.
LI_EXPORT int li_scan_carry(float* state, long long state_stride, float* chunk_state, const float* chunk_decay, const float* token_decay,
                            const int* seg, const int* runs, int nruns, int heads, int per_head, int period, cudaStream_t stream) {
    LI_REQUIRE(heads > 0 && per_head > 0, "scan carry: %d heads of %d elements", heads, per_head);
    LI_REQUIRE(period >= 0 && (period == 0 || (chunk_decay != nullptr && per_head % period == 0)), "scan carry: %d decays a head for %d elements", period, per_head);
    LI_REQUIRE(chunk_decay != nullptr || (token_decay != nullptr && seg != nullptr), "scan carry: no decay given");
    if (nruns == 0) return 0;
    LI_REQUIRE(nruns <= 65535, "scan carry: %d sequences in one launch", nruns);
    cudaError_t e = li_launch_pdl(scan_carry_kernel, dim3(ceil_div(heads * per_head, 256), nruns), dim3(256), 0, stream, state, state_stride, chunk_state,
                                  chunk_decay, token_decay, seg, runs, heads, per_head, period);
    if (e != cudaSuccess) return li_fail("scan_carry: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("scan_carry");
}

LI_EXPORT int li_gated_rmsnorm(const float* y, const void* gate, int dtype, int gate_stride, int gate_off, const float* w, float eps, int mode,
                               void* out, int T, int n, int groups, cudaStream_t stream) {
    LI_REQUIRE(n > 0 && groups > 0 && n % groups == 0, "gated norm: %d columns in %d groups", n, groups);
    LI_REQUIRE(mode >= 0 && mode <= 2, "gated norm: unknown mode %d", mode);
    LI_REQUIRE(gate_off >= 0 && gate_off + n <= gate_stride, "gated norm: gate at column %d of %d for %d columns", gate_off, gate_stride, n);
    if (T == 0) return 0;
    const long long blocks = (long long)T * groups;
    LI_REQUIRE(blocks < (1LL << 31), "gated norm: too many rows");
    cudaError_t e;
    if (n / groups <= kWarpGroup && (dtype == LI_F32 || dtype == LI_BF16)) {
        const dim3 grid((unsigned)((blocks + 7) / 8));
        const int gsz = n / groups;
        const bool vec4 = gsz % 4 == 0 && gate_stride % 4 == 0 && gate_off % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)gate % 16 == 0 &&
                          (uintptr_t)out % 16 == 0;
#define LI_NORM(TT, VV)                                                                                                                        \
    e = li_launch_pdl(gated_rmsnorm_warp_kernel<TT, VV>, grid, dim3(256), 0, stream, y, (const TT*)gate, gate_stride, gate_off, w, eps, mode, (TT*)out, n, \
                      groups, blocks)
        if (dtype == LI_F32) {
            if (vec4) LI_NORM(float, true); else LI_NORM(float, false);
        } else {
            if (vec4) LI_NORM(bf16, true); else LI_NORM(bf16, false);
        }
#undef LI_NORM
        if (e != cudaSuccess) return li_fail("gated_rmsnorm: launch failed: %s", cudaGetErrorString(e));
        return li_check_launch("gated_rmsnorm");
    }
    if (dtype == LI_F32)
        e = li_launch_pdl(gated_rmsnorm_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, y, (const float*)gate, gate_stride, gate_off, w, eps,
                          mode, (float*)out, n, groups);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(gated_rmsnorm_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, y, (const bf16*)gate, gate_stride, gate_off, w, eps,
                          mode, (bf16*)out, n, groups);
    else
        return li_fail("gated norm: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("gated_rmsnorm: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("gated_rmsnorm");
}
