// Products in groups, and the routing of a mixture of experts around them.
//
//   li_grouped_linear: G products out_g = a_g w_g^T with one matrix w_g [N, K] per group (w is [G, N, K]), two ways:
//     * rows in groups (row_offsets [G + 1] on the device): group g owns the rows row_offsets[g] .. row_offsets[g + 1] - 1 of
//       a [M, lda] and of out [M, ldc], all columns alike: the experts of a mixture, tokens sorted by expert;
//     * columns in groups (row_offsets NULL): every group takes all M rows, its inputs at column g * a_gcol of a and its
//       outputs at column g * c_gcol of out: a map per head.
//     float32 (and bfloat16 shapes the other kernel refuses): CUDA-core tiles of 64 x 64 x 16.  bfloat16 with K a
//     multiple of 8: mma.sync tiles of 64 x 64 (many rows a group) or 16 x 64 (few: the weights are what is read; four
//     stages), operands through shared memory with 16-byte asynchronous copies; rows in groups whose runs are padded to
//     128 rows and number 256 or more go to tcgen05 tiles (gemm_tcgen05.cu).  Either way float accumulation, each output summed over k in ascending
//     order by one thread: a row's result does not depend on which rows stand beside it.
//   li_moe_route:   scores = sigmoid(logits), the `top` largest per token (the lower index wins a tie); the scores of the
//     chosen are the weights as they are, not renormalised.  Or the largest logits choose, and the weights are the softmax
//     over the chosen logits alone.
//   li_moe_sort:    a stable counting sort of the (token, choice) pairs by expert: offsets per expert, the pair at each
//     sorted place, and each pair's place.  One block per expert walks the pairs in order, so the result is the same
//     whatever runs beside it.
//   li_moe_gather:  sorted row r = weight(pair) * h[token(pair)] (the weight goes on the expert's input), or the plain row.
//   li_moe_combine: y[t] = sum over the token's choices of the sorted rows (times the weight, when it goes on the output),
//     summed in float in the order of the choices.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const Tin* __restrict__ A, int lda, int a_gcol, const Tin* __restrict__ W, Tout* __restrict__ C, int ldc, int c_gcol,
                      const int* __restrict__ row_offsets, int M, int N, int K, int G) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (row_offsets) {
        // blockIdx.y counts row tiles over all groups: find the group this one falls into
        int tile = blockIdx.y;
        g = 0;
        while (g < G) {
            const int rows = row_offsets[g + 1] - row_offsets[g];
            const int tiles = (rows + BM - 1) / BM;
            if (tile < tiles) break;
            tile -= tiles;
            ++g;
        }
        if (g >= G) return;
        m0 = row_offsets[g] + tile * BM;
        m_end = row_offsets[g + 1];
    } else {
        g = blockIdx.z;
        m0 = blockIdx.y * BM;
        m_end = M;
    }
    const Tin* a = A + (size_t)g * a_gcol;
    const Tin* w = W + (size_t)g * N * K;
    Tout* c = C + (size_t)g * c_gcol;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * BN;
    const int tx = tid & 15, ty = tid >> 4;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lr, wn = n0 + lr;
            av[q] = (am < m_end && k < K) ? to_float(a[(size_t)am * lda + k]) : 0.0f;
            wv[q] = (wn < N && k < K) ? to_float(w[(size_t)wn * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            As[lk + q][lr] = av[q];
            Ws[lk + q][lr] = wv[q];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float ar[TM], wr[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ar[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wr[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= m_end) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) c[(size_t)m * ldc + n] = from_float<Tout>(acc[i][j]);
        }
    }
}

// ---- the same on the tensor cores (bfloat16) ----------------------------------------------------------------------------

constexpr int MPAD = 8;                   // padding of a shared row: rows of TK + 8 elements keep 16-byte alignment and spread over the banks

__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                               // 0: the destination is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A tile of TM rows x 64 columns a CTA of four warps, TK elements of k a stage, ST stages of 16-byte asynchronous copies.
// TM 64: many rows a group (portions of prompts); a warp takes 16 rows and all 64 columns.  TM 16: few rows a group
// (single tokens: the weights are what is read): a warp takes all 16 rows and 16 of the columns, and four stages of
// 64 elements keep more of the weights on their way.
// kSwiglu (1, or 2: the gated unit with bounded operands, glu_params = {limit, alpha} on the device): the columns come as 8 gate,
// 8 up, 8 gate, 8 up, ... (the rows of every group's matrix interleaved in eights), and out [M, N / 2] takes
// up * gate / (1 + exp(-gate)) (or the bounded unit): a thread holds a gate column and its up column in neighbouring tiles of 8.
template <int TM, int TK, int ST, int kSwiglu>
__global__ void __launch_bounds__(128)
grouped_mma_kernel(const bf16* __restrict__ A, int lda, int a_gcol, const bf16* __restrict__ W, bf16* __restrict__ C, int ldc, int c_gcol,
                   const int* __restrict__ row_offsets, int M, int N, int K, int G, const float* __restrict__ glu_params) {
    __shared__ __align__(16) bf16 As[ST][TM][TK + MPAD];
    __shared__ __align__(16) bf16 Ws[ST][BN][TK + MPAD];
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (row_offsets) {
        int tile = blockIdx.y;
        g = 0;
        while (g < G) {
            const int rows = row_offsets[g + 1] - row_offsets[g];
            const int tiles = (rows + TM - 1) / TM;
            if (tile < tiles) break;
            tile -= tiles;
            ++g;
        }
        if (g >= G) return;
        m0 = row_offsets[g] + tile * TM;
        m_end = row_offsets[g + 1];
    } else {
        g = blockIdx.z;
        m0 = blockIdx.y * TM;
        m_end = M;
    }
    const bf16* a = A + (size_t)g * a_gcol;
    const bf16* w = W + (size_t)g * N * K;
    bf16* c = C + (size_t)g * c_gcol;
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, t = lane & 3;
    constexpr int CH = TK / 8;                                      // 16-byte chunks of a row of a stage
    auto load = [&](int stage, int k0) {
        for (int idx = tid; idx < TM * CH; idx += 128) {
            const int r = idx / CH, ch = idx - r * CH;
            const int k = k0 + ch * 8;
            const bool v = k < K && m0 + r < m_end;
            cp16(&As[stage][r][ch * 8], v ? a + (size_t)(m0 + r) * lda + k : a, v);
        }
        for (int idx = tid; idx < BN * CH; idx += 128) {
            const int r = idx / CH, ch = idx - r * CH;
            const int k = k0 + ch * 8;
            const bool v = k < K && n0 + r < N;
            cp16(&Ws[stage][r][ch * 8], v ? w + (size_t)(n0 + r) * K + k : w, v);
        }
    };
    constexpr int NT = TM == 64 ? 8 : 2;                            // tiles of 8 columns a warp
    const int row0 = TM == 64 ? warp * 16 : 0, col0 = TM == 64 ? 0 : warp * 16;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    const int nk = (K + TK - 1) / TK;
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) {
        if (s < nk) load(s, s * TK);
        asm volatile("cp.async.commit_group;");
    }
    for (int kb = 0; kb < nk; ++kb) {
        asm volatile("cp.async.wait_group %0;" ::"n"(ST - 2));
        __syncthreads();                     // stage kb has landed for everybody, and everybody is done with the stage that is loaded next
        if (kb + ST - 1 < nk) load((kb + ST - 1) % ST, (kb + ST - 1) * TK);
        asm volatile("cp.async.commit_group;");
        const int stage = kb % ST;
#pragma unroll
        for (int ks = 0; ks < TK; ks += 16) {
            const bf16* ar = &As[stage][row0 + gq][ks + 2 * t];
            const unsigned a0 = *reinterpret_cast<const unsigned*>(ar), a1 = *reinterpret_cast<const unsigned*>(ar + 8 * (TK + MPAD));
            const unsigned a2 = *reinterpret_cast<const unsigned*>(ar + 8), a3 = *reinterpret_cast<const unsigned*>(ar + 8 * (TK + MPAD) + 8);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bf16* wr = &Ws[stage][col0 + j * 8 + gq][ks + 2 * t];
                mma16816(acc[j], a0, a1, a2, a3, *reinterpret_cast<const unsigned*>(wr), *reinterpret_cast<const unsigned*>(wr + 8));
            }
        }
    }
    const int r_lo = m0 + row0 + gq, r_hi = r_lo + 8;
    if constexpr (kSwiglu) {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
            const int gate_col = n0 + col0 + j * 8 + 2 * t;           // its up column stands 8 further on
            const int n = (n0 + col0 + j * 8) / 2 + 2 * t;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (gate_col + i + 8 < N) {
                    if (r_lo < m_end) c[(size_t)r_lo * ldc + n + i] = __float2bfloat16_rn(glu_of<bf16, kSwiglu == 2>(acc[j][i], acc[j + 1][i], glu_params));
                    if (r_hi < m_end) c[(size_t)r_hi * ldc + n + i] = __float2bfloat16_rn(glu_of<bf16, kSwiglu == 2>(acc[j][2 + i], acc[j + 1][2 + i], glu_params));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int n = n0 + col0 + j * 8 + 2 * t;
        if (n < N) {
            if (r_lo < m_end) c[(size_t)r_lo * ldc + n] = __float2bfloat16_rn(acc[j][0]);
            if (r_hi < m_end) c[(size_t)r_hi * ldc + n] = __float2bfloat16_rn(acc[j][2]);
        }
        if (n + 1 < N) {
            if (r_lo < m_end) c[(size_t)r_lo * ldc + n + 1] = __float2bfloat16_rn(acc[j][1]);
            if (r_hi < m_end) c[(size_t)r_hi * ldc + n + 1] = __float2bfloat16_rn(acc[j][3]);
        }
    }
}

// ---- routing ---------------------------------------------------------------------------------------------------------

constexpr int kMaxExpertsPerLane = 8;       // experts <= 256

__global__ void moe_route_kernel(const float* __restrict__ logits, int scoring, int T, int E, int top, int* __restrict__ ids,
                                 float* __restrict__ weights) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float s[kMaxExpertsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        const float z = e < E ? logits[(size_t)t * E + e] : 0.0f;
        // sigmoid scores lie in (0, 1): -1 never wins; logits taken as they are: the lowest float never wins
        if (scoring == 0) s[i] = e < E ? 1.0f / (1.0f + expf(-z)) : -1.0f;
        else s[i] = e < E ? fmaxf(z, -3.0e38f) : -3.4e38f;
    }
    const float gone = scoring == 0 ? -1.0f : -3.4e38f;
    for (int k = 0; k < top; ++k) {
        float best = scoring == 0 ? -2.0f : -INFINITY;
        int arg = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (s[i] > best) best = s[i], arg = e;                 // ascending e within a lane: the lower index keeps a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
        }
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = best;
        }
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (lane + 32 * i == arg) s[i] = gone;
    }
    if (scoring == 1 && lane == 0) {
        // the weights are the softmax over the chosen logits alone (the first chosen is the largest)
        float* wt = weights + (size_t)t * top;
        const float m = wt[0];
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) sum += expf(wt[k] - m);
        for (int k = 0; k < top; ++k) wt[k] = expf(wt[k] - m) / sum;
    }
}

// Routing over all experts at once with groups: scores s = softmax(logits) over the E outputs; the choice scores are
// s + correction; the experts form `groups` equal groups of neighbours, a group's score is its largest choice score, and only
// experts of the `keep` best groups can be chosen (the lower index wins a tie, among groups and among experts); the `top`
// largest choice scores choose; the weights are the chosen experts' s (without the correction), divided by their sum + 1e-20,
// times `scale`.  One warp a token, everything in float.
__global__ void moe_route_grouped_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int T, int E, int top, int groups,
                                         int keep, float scale, int* __restrict__ ids, float* __restrict__ weights) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float s[kMaxExpertsPerLane], c[kMaxExpertsPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
        m = fmaxf(m, s[i]);
    }
    m = warp_max(m);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        s[i] = lane + 32 * i < E ? expf(s[i] - m) : 0.0f;
        sum += s[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = s[i] / sum;
        c[i] = e < E ? s[i] + (correction ? correction[e] : 0.0f) : -INFINITY;
    }
    const int per = E / groups;
    if (keep < groups) {
        // the groups' scores, then `keep` rounds that each take the best group left; an expert stays if its group was taken
        unsigned taken[kMaxExpertsPerLane];                     // per expert of this lane: its group is among the kept ones
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) taken[i] = 0u;
        for (int round = 0; round < keep; ++round) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < kMaxExpertsPerLane; ++i) {
                const int e = lane + 32 * i;
                if (e < E && !taken[i]) {
                    const int g = e / per;
                    if (c[i] > best || (c[i] == best && g < arg)) best = c[i], arg = g;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
            }
#pragma unroll
            for (int i = 0; i < kMaxExpertsPerLane; ++i) {
                const int e = lane + 32 * i;
                if (e < E && e / per == arg) taken[i] = 1u;
            }
        }
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (!taken[i]) c[i] = -INFINITY;
    }
    float wsum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, score = 0.0f;
        int arg = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (c[i] > best || (arg == 0x7fffffff && c[i] == best))) best = c[i], arg = e, score = s[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            const float os = __shfl_xor_sync(0xffffffffu, score, o);
            if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa, score = os;
        }
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = score;
        }
        wsum += score;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (lane + 32 * i == arg) c[i] = -INFINITY, s[i] = 0.0f;
    }
    if (lane == 0) {
        float* wt = weights + (size_t)t * top;
        for (int k = 0; k < top; ++k) wt[k] = wt[k] / (wsum + 1e-20f) * scale;
    }
}

// One block per expert.  n pairs (token, choice) in order; ids[i] is pair i's expert.  Every expert's run of rows starts
// at a multiple of `pad` (1: runs follow one another closely); the places between a run's last pair and the next run
// hold no pair (-1).  tile_group (may be NULL; pad > 1): for every tile of `pad` rows, the expert it belongs to, -1 behind the last run.
// Experts from `matrices` on have no matrices (their rows pass as they are): their tiles belong to no group either (-1).
__global__ void moe_sort_kernel(const int* __restrict__ ids, int n, int E, int matrices, int pad, int* __restrict__ offsets, int* __restrict__ pair_at,
                                int* __restrict__ place_of, int* __restrict__ tile_group, int n_tiles, int places) {
    __shared__ int warp_total[32];
    __shared__ int hist[kMaxExpertsPerLane * 32];
    __shared__ int base_eq;
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // how many pairs go to every expert (integer sums: the same whatever the order), then where this expert's rows start
    for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    if (threadIdx.x == 0) base_eq = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int id = ids[i];
        if (id >= 0 && id < E) atomicAdd(&hist[id], 1);
    }
    __syncthreads();
    int start = 0;
    for (int x = 0; x < e; ++x) start += (hist[x] + pad - 1) / pad * pad;
    const int mine_total = hist[e];
    const int end = start + (mine_total + pad - 1) / pad * pad;
    // this expert's pairs, in order
    for (int base = 0; base < n; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const bool mine = i < n && ids[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_total[warp] = __popc(ballot);
        __syncthreads();
        int before = base_eq;
        for (int w = 0; w < warp; ++w) before += warp_total[w];
        if (mine) {
            const int place = start + before + __popc(ballot & ((1u << lane) - 1u));
            pair_at[place] = i;
            place_of[i] = place;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < nwarps; ++w) total += warp_total[w];
            base_eq += total;
        }
        __syncthreads();
    }
    for (int r = start + mine_total + threadIdx.x; r < end; r += blockDim.x) pair_at[r] = -1;
    if (e == E - 1)
        for (int r = end + threadIdx.x; r < places; r += blockDim.x) pair_at[r] = -1;          // places behind the last run belong to nobody
    if (tile_group != nullptr) {
        for (int tl = start / pad + threadIdx.x; tl < end / pad && tl < n_tiles; tl += blockDim.x) tile_group[tl] = e < matrices ? e : -1;
        if (e == E - 1)
            for (int tl = end / pad + threadIdx.x; tl < n_tiles; tl += blockDim.x) tile_group[tl] = -1;
    }
    if (threadIdx.x == 0) {
        offsets[e] = start;
        if (e == E - 1) offsets[E] = end;
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ pair_at, const float* __restrict__ weights, int top, int H,
                                  T* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int pair = pair_at[r];
    T* dst = out + (size_t)r * H;
    if (pair < 0) {                                        // a place between two experts' runs: a row of zeros
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_float<T>(0.0f);
        return;
    }
    const T* src = h + (size_t)(pair / top) * H;
    if (weights) {
        const float w = weights[pair];
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_float<T>(w * to_float(src[i]));
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place_of, const float* __restrict__ weights, int top, int H,
                                   T* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < top; ++k) {
            const float v = to_float(rows[(size_t)place_of[(size_t)t * top + k] * H + i]);
            acc += weights ? weights[(size_t)t * top + k] * v : v;
        }
        y[(size_t)t * H + i] = from_float<T>(acc);
    }
}

}  // namespace

int li_linear_tcgen05_grouped(const void* a, const void* w, void* out, int M, int N, int K, int G, const int* tile_group, int epilogue,
                              const float* glu_params, cudaStream_t stream);

// tile_group (may be NULL; rows in groups whose runs start at multiples of 128, li_moe_sort with pad 128): the group of
// every tile of 128 rows; bfloat16 products of at least kTensorRows rows then run on tcgen05 tiles.
constexpr int kTensorRows = 256;

// epilogue: LI_EPILOGUE_NONE, or a gated one (bfloat16, K a multiple of 8, N a multiple of 16): gate and up rows of
// every group's matrix interleaved in eights, out rows of N / 2 activations; LI_EPILOGUE_GLU_CLAMPED reads its {limit, alpha}
// from glu_params on the device.
LI_EXPORT int li_grouped_linear(const void* a, int lda, int a_gcol, const void* w, void* out, int ldc, int c_gcol, const int* row_offsets,
                                const int* tile_group, int dtype, int M, int N, int K, int G, int epilogue, const float* glu_params,
                                cudaStream_t stream) {
    LI_REQUIRE(M >= 0 && N > 0 && K > 0 && G > 0, "grouped_linear: bad sizes M=%d N=%d K=%d G=%d", M, N, K, G);
    LI_REQUIRE(epilogue == LI_EPILOGUE_NONE || li_epilogue_is_gated(epilogue), "grouped_linear: unknown epilogue %d", epilogue);
    LI_REQUIRE(li_epilogue_bias_ok(epilogue, glu_params) || epilogue == LI_EPILOGUE_NONE, "grouped_linear: the bounded unit needs its parameters, the others take none");
    const bool swiglu = li_epilogue_is_gated(epilogue);
    const bool clamped = epilogue == LI_EPILOGUE_GLU_CLAMPED;
    const int out_cols = swiglu ? N / 2 : N;
    LI_REQUIRE(lda >= K && ldc >= out_cols, "grouped_linear: rows of %d and %d elements cannot hold K=%d and %d outputs", lda, ldc, K, out_cols);
    LI_REQUIRE(row_offsets == nullptr || (a_gcol == 0 && c_gcol == 0), "grouped_linear: groups are rows or columns, not both");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "grouped_linear: unknown dtype %d", dtype);
    if (M == 0) return 0;
    if (dtype == LI_BF16 && row_offsets != nullptr && tile_group != nullptr && M >= kTensorRows && M % 128 == 0 && lda == K && ldc == out_cols &&
        K % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0 && (!swiglu || N % 16 == 0))
        return li_linear_tcgen05_grouped(a, w, out, M, N, K, G, tile_group, epilogue, glu_params, stream);
    const int row_tiles = ceil_div(M, BM);
    const dim3 grid(ceil_div(N, BN), row_offsets ? row_tiles + G : row_tiles, row_offsets ? 1 : G);
    LI_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "grouped_linear: too many tiles for one launch");
    cudaError_t e;
    // 16-byte copies: every row and every group's first column on a 16-byte boundary
    const bool aligned = K % 8 == 0 && lda % 8 == 0 && a_gcol % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0;
    LI_REQUIRE(!swiglu || (dtype == LI_BF16 && aligned && N % 16 == 0), "grouped_linear: the swiglu epilogue takes bfloat16, K a multiple of 8 and N a multiple of 16");
    // few rows a group (single tokens): tiles of 16 rows, more of the weights in flight
    const bool few = row_offsets ? M <= 32 * G : M <= 32;
    if (dtype == LI_BF16 && aligned && few) {
        const int tiles16 = ceil_div(M, 16);
        const dim3 grid16(ceil_div(N, BN), row_offsets ? tiles16 + G : tiles16, row_offsets ? 1 : G);
#define LI_GROUPED_MMA(TM_, TK_, ST_, EPI_, GRID_)                                                                                          \
    li_launch_pdl(grouped_mma_kernel<TM_, TK_, ST_, EPI_>, GRID_, dim3(128), 0, stream, (const bf16*)a, lda, a_gcol, (const bf16*)w, (bf16*)out, ldc, \
                  c_gcol, row_offsets, M, N, K, G, glu_params)
        e = clamped ? LI_GROUPED_MMA(16, 64, 4, 2, grid16) : swiglu ? LI_GROUPED_MMA(16, 64, 4, 1, grid16) : LI_GROUPED_MMA(16, 64, 4, 0, grid16);
    } else if (dtype == LI_BF16 && aligned)
        e = clamped ? LI_GROUPED_MMA(64, 32, 3, 2, grid) : swiglu ? LI_GROUPED_MMA(64, 32, 3, 1, grid) : LI_GROUPED_MMA(64, 32, 3, 0, grid);
#undef LI_GROUPED_MMA
    else if (dtype == LI_F32)
        e = li_launch_pdl(grouped_linear_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)a, lda, a_gcol, (const float*)w, (float*)out,
                          ldc, c_gcol, row_offsets, M, N, K, G);
    else
        e = li_launch_pdl(grouped_linear_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)a, lda, a_gcol, (const bf16*)w, (bf16*)out, ldc,
                          c_gcol, row_offsets, M, N, K, G);
    if (e != cudaSuccess) return li_fail("grouped_linear: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("grouped_linear");
}

// scoring 0: the scores are sigmoid(logits) and the chosen experts' scores are their weights; 1: the largest logits choose and
// the weights are the softmax over the chosen logits alone.
LI_EXPORT int li_moe_route(const float* logits, int scoring, int T, int E, int top, int* ids, float* weights, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && E > 0 && top > 0 && top <= E, "moe_route: %d of %d experts", top, E);
    LI_REQUIRE(scoring == 0 || scoring == 1, "moe_route: unknown scoring %d", scoring);
    LI_REQUIRE(E <= 32 * kMaxExpertsPerLane, "moe_route: %d experts are more than %d", E, 32 * kMaxExpertsPerLane);
    if (T == 0) return 0;
    const cudaError_t e = li_launch_pdl(moe_route_kernel, dim3(ceil_div(T, 4)), dim3(128), 0, stream, logits, scoring, T, E, top, ids, weights);
    if (e != cudaSuccess) return li_fail("moe_route: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_route");
}

// See moe_route_grouped_kernel.  correction (may be NULL): [E] float; groups divides E; 1 <= keep <= groups; the kept groups
// must hold at least `top` experts.
LI_EXPORT int li_moe_route_grouped(const float* logits, const float* correction, int T, int E, int top, int groups, int keep, float scale, int* ids,
                                   float* weights, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && E > 0 && top > 0 && top <= E, "moe_route_grouped: %d of %d experts", top, E);
    LI_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && keep * (E / groups) >= top,
               "moe_route_grouped: %d of %d groups of %d experts cannot give %d choices", keep, groups, groups >= 1 ? E / groups : 0, top);
    LI_REQUIRE(E <= 32 * kMaxExpertsPerLane, "moe_route_grouped: %d experts are more than %d", E, 32 * kMaxExpertsPerLane);
    if (T == 0) return 0;
    const cudaError_t e = li_launch_pdl(moe_route_grouped_kernel, dim3(ceil_div(T, 4)), dim3(128), 0, stream, logits, correction, T, E, top, groups, keep,
                                        scale, ids, weights);
    if (e != cudaSuccess) return li_fail("moe_route_grouped: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_route_grouped");
}

// pad: every expert's run of rows starts at a multiple of it; pair_at has `places` entries, room for n + E (pad - 1) of them,
// and tile_group (may be NULL) one entry for each of its n_tiles tiles of pad rows.
LI_EXPORT int li_moe_sort(const int* ids, int n, int E, int matrices, int pad, int* offsets, int* pair_at, int* place_of, int* tile_group, int n_tiles,
                          int places, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && E > 0 && pad >= 1 && matrices >= 0 && matrices <= E, "moe_sort: bad sizes");
    LI_REQUIRE(places >= n + (pad > 1 ? E * (pad - 1) : 0), "moe_sort: %d places cannot hold %d pairs in runs padded to %d", places, n, pad);
    LI_REQUIRE(E <= 32 * kMaxExpertsPerLane, "moe_sort: %d experts are more than %d", E, 32 * kMaxExpertsPerLane);
    const cudaError_t e = li_launch_pdl(moe_sort_kernel, dim3(E), dim3(256), 0, stream, ids, n, E, matrices, pad, offsets, pair_at, place_of, tile_group, n_tiles, places);
    if (e != cudaSuccess) return li_fail("moe_sort: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_sort");
}

// out [n, H]: row r is h[pair_at[r] / top], times weights[pair_at[r]] if weights is given; zeros where pair_at[r] < 0.
LI_EXPORT int li_moe_gather(const void* h, int dtype, const int* pair_at, const float* weights, int n, int top, int H, void* out, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && top > 0 && H > 0, "moe_gather: bad sizes");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "moe_gather: unknown dtype %d", dtype);
    if (n == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(moe_gather_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)h, pair_at, weights, top, H, (float*)out);
    else
        e = li_launch_pdl(moe_gather_kernel<bf16>, dim3(n), dim3(threads), 0, stream, (const bf16*)h, pair_at, weights, top, H, (bf16*)out);
    if (e != cudaSuccess) return li_fail("moe_gather: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_gather");
}

// y [T, H]: y[t] = sum_k rows[place_of[t * top + k]] (times weights[t * top + k] if weights is given).
LI_EXPORT int li_moe_combine(const void* rows, int dtype, const int* place_of, const float* weights, int T, int top, int H, void* y,
                             cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && top > 0 && H > 0, "moe_combine: bad sizes");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "moe_combine: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)rows, place_of, weights, top, H, (float*)y);
    else
        e = li_launch_pdl(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)rows, place_of, weights, top, H, (bf16*)y);
    if (e != cudaSuccess) return li_fail("moe_combine: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_combine");
}
