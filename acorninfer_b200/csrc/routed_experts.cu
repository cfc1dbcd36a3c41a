// A routed mixture of experts: the router's choice, the grouping of tokens by expert, a matrix
// product per expert over its tokens, and the weighted sum.
//
//   moe_route     per token: s = softmax(z) over all N router outputs; the choice score is s + correction;
//                 the outputs form `groups` equal groups of neighbours, a group's score is its largest choice
//                 score, and only outputs of the `keep` best groups can be chosen; the `top` largest choice
//                 scores win; their weights are s itself, or with `normalize` s over the chosen's sum
//                 (+ 1e-20).  float32 throughout.
//   moe_plan      counts per expert, offsets (exclusive sums) and a slot for every (token, choice) pair,
//                 so that the pairs of an expert are neighbours: slot_token[slot], slot_of[pair].
//   grouped_gemm  C[slot, :] = A[row(slot), :] W_e^T for the slots of every expert e < E
//   moe_combine   out[t] = sum_k weight_k * (chosen_k >= E ? x[t] : y[slot_of(t, k)]) (+ extra[t], if given)
//                 (router outputs from E on are identity experts: they return their input)
#include "mma_helpers.cuh"

// One warp per token.  Ties go to the lower index.
__global__ void moe_route_kernel(const float* __restrict__ z, const float* __restrict__ correction,
                                 int* __restrict__ idx, float* __restrict__ wts, int tokens, int N, int top, int groups,
                                 int keep, int normalize) {
    extern __shared__ float sm[];                       // per warp: s[N], choice[N]
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float* s = sm + (size_t)warp * 2 * N;
    float* choice = s + N;
    const float* zr = z + (int64_t)t * N;
    float m = -INFINITY;
    for (int i = lane; i < N; i += 32) m = fmaxf(m, zr[i]);
    m = warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < N; i += 32) {
        const float e = expf(zr[i] - m);
        s[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int i = lane; i < N; i += 32) {
        s[i] = s[i] / sum;
        choice[i] = s[i] + correction[i];
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // the `keep` groups with the largest best choice score, found one by one; a bit per kept group
        const int per = N / groups;
        unsigned long long kept_lo = 0ull;              // groups <= 64: bit per kept group
        for (int round = 0; round < keep; ++round) {
            float best = -INFINITY;
            int best_g = groups;
            for (int gi = lane; gi < groups; gi += 32) {
                if ((kept_lo >> gi) & 1ull) continue;
                float gm = -INFINITY;
                for (int i = gi * per; i < (gi + 1) * per; ++i) gm = fmaxf(gm, choice[i]);
                if (gm > best || (gm == best && gi < best_g)) {
                    best = gm;
                    best_g = gi;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (ob > best || (ob == best && og < best_g)) {
                    best = ob;
                    best_g = og;
                }
            }
            if (best_g < groups) kept_lo |= 1ull << best_g;
        }
        for (int i = lane; i < N; i += 32)
            if (!((kept_lo >> (i / per)) & 1ull)) choice[i] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_i = N;
        for (int i = lane; i < N; i += 32) {
            const float c = choice[i];
            if (c > best || (c == best && i < best_i && c > -INFINITY)) {
                best = c;
                best_i = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) {
                best = ob;
                best_i = oi;
            }
        }
        if (best_i >= N) best_i = 0;                    // nothing left to choose (top > allowed outputs): weight 0
        if (lane == 0) {
            idx[(int64_t)t * top + k] = best_i;
            wts[(int64_t)t * top + k] = best > -INFINITY ? s[best_i] : 0.f;
            choice[best_i] = -INFINITY;
        }
        __syncwarp();
    }
    if (normalize && lane == 0) {
        float total = 0.f;
        for (int k = 0; k < top; ++k) total += wts[(int64_t)t * top + k];
        total += 1e-20f;
        for (int k = 0; k < top; ++k) wts[(int64_t)t * top + k] /= total;
    }
}

extern "C" int acorn_moe_route(const float* z, const float* correction, int* idx, float* wts, int tokens, int N, int top,
                               int groups, int keep, int normalize, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (N < 1 || top < 1 || top > N || groups < 1 || groups > 64 || N % groups || keep < 1 || keep > groups || N > 2048)
        return ACORN_ERR_UNSUPPORTED;
    const int warps = 4;
    const size_t smem = (size_t)warps * 2 * N * sizeof(float);
    static AcornPerDevice configured;
    if (smem > 48 * 1024 && !configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * 2048 * 4);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    return acorn_launch(moe_route_kernel, dim3((tokens + warps - 1) / warps), dim3(32 * warps), smem, stream, z, correction,
                        idx, wts, tokens, N, top, groups, keep, normalize);
}

// One block: histogram of the chosen outputs, exclusive sums, then a slot for every pair.  Within an
// expert the slots are handed out in whatever order the threads arrive: a row's result does not
// depend on its slot.
__global__ void moe_plan_kernel(const int* __restrict__ idx, int* __restrict__ offsets, int* __restrict__ slot_of,
                                int* __restrict__ slot_token, int pairs, int N, int top) {
    extern __shared__ int cnt[];                        // [N] counts, then [N] cursors
    pdl_wait();
    pdl_trigger();
    int* cursor = cnt + N;
    for (int i = threadIdx.x; i < N; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < N; ++i) {
            offsets[i] = run;
            cursor[i] = run;
            run += cnt[i];
        }
        offsets[N] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int slot = atomicAdd(&cursor[idx[i]], 1);
        slot_of[i] = slot;
        slot_token[slot] = i / top;
    }
}

extern "C" int acorn_moe_plan(const int* idx, int* offsets, int* slot_of, int* slot_token, int pairs, int N, int top,
                              cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (N > 4096) return ACORN_ERR_UNSUPPORTED;
    return acorn_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * N * sizeof(int), stream, idx, offsets, slot_of,
                        slot_token, pairs, N, top);
}

// out[i, :] = x[rows[i], :]: the tokens' rows in the order of the slots, for a product whose operand tiles are
// fetched by TMA (contiguous rows).  16 bytes a thread and step when the rows allow it.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ rows, T* __restrict__ out, int H) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = blockIdx.x;
    const T* src = x + (int64_t)rows[i] * H;
    T* dst = out + i * H;
    constexpr int EPC = 16 / (int)sizeof(T);
    if (H % EPC == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        for (int c = threadIdx.x; c < H / EPC; c += blockDim.x)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
    }
}

extern "C" int acorn_gather_rows(const void* x, const int* rows, void* out, int n, int H, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(gather_rows_kernel<T>, dim3(n), dim3(128), 0, stream, (const T*)x, rows,
                                                       (T*)out, H));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- a product per expert
// Slots offsets[e] .. offsets[e+1]-1 belong to expert e.  Row `slot` of A is a_rows ? A[a_rows[slot]] : A[slot].
// A block finds its (expert, tile of GG_BM slots) by walking the offsets; blocks beyond the last tile
// leave.  float32 accumulation, one chain over k = 0, 1, ... per output.
#define GG_BM 32
#define GG_BN 64
#define GG_BK 32

template <typename T>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const T* __restrict__ A, int64_t lda, const int* __restrict__ a_rows,
                                                           const T* __restrict__ W, T* __restrict__ C, int64_t ldc,
                                                           const int* __restrict__ offsets, int E, int N, int K) {
    __shared__ float as[GG_BM][GG_BK + 1];
    __shared__ float ws[GG_BN][GG_BK + 1];
    __shared__ int s_e, s_first, s_end;
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, e = 0, found = -1;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + GG_BM - 1) / GG_BM;
            if (tile < tiles) {
                found = e;
                break;
            }
            tile -= tiles;
        }
        s_e = found;
        if (found >= 0) {
            s_first = offsets[found] + tile * GG_BM;
            s_end = offsets[found + 1];
        }
    }
    __syncthreads();
    const int e = s_e;
    if (e < 0) return;
    const int first = s_first, end = s_end;
    const int n0 = blockIdx.x * GG_BN;
    const T* We = W + (int64_t)e * N * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 column groups of 4, 16 row pairs
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int i = threadIdx.x; i < GG_BM * GG_BK; i += 256) {
            const int rr = i / GG_BK, kk = i % GG_BK;
            const int slot = first + rr, k = k0 + kk;
            float v = 0.f;
            if (slot < end && k < K) {
                const int64_t row = a_rows ? a_rows[slot] : slot;
                v = to_float(A[row * lda + k]);
            }
            as[rr][kk] = v;
        }
        for (int i = threadIdx.x; i < GG_BN * GG_BK; i += 256) {
            const int nn = i / GG_BK, kk = i % GG_BK;
            const int n = n0 + nn, k = k0 + kk;
            ws[nn][kk] = (n < N && k < K) ? to_float(We[(int64_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            const float a0 = as[ty][kk], a1 = as[ty + 16][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float w = ws[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, w, acc[0][j]);
                acc[1][j] = fmaf(a1, w, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int slot = first + ty + 16 * i;
        if (slot >= end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n < N) C[(int64_t)slot * ldc + n] = from_float<T>(acc[i][j]);
        }
    }
}

// ---------------------------------------------------------------- the same on the tensor cores (bfloat16)
// mma.sync m16n8k16, float32 accumulation in the order of K.  A block: BM slots of one expert by 128
// weight rows; eight warps; operand tiles of 64 along K through a ring of cp.async stages.  BM = 128 or 64
// (warps 2 x 4, 64 x 32 or 32 x 32 each) for steps with many rows an expert, BM = 16 (warps 1 x 8, 16 x 16 each) for
// decode steps, where the kernel is bound by reading every chosen expert's matrix once.  An output
// element is the same chain of products in both, so a row's bits do not depend on the step it is in.
#define GT_BN 128
#define GT_BK 64
#define GT_LDS (GT_BK + 8)
#define GT_STAGES 3

template <int BM>
__global__ void __launch_bounds__(256) grouped_gemm_tc_kernel(const bf16* __restrict__ A, int64_t lda,
                                                              const int* __restrict__ a_rows, const bf16* __restrict__ W,
                                                              bf16* __restrict__ C, int64_t ldc,
                                                              const int* __restrict__ offsets, int E, int N, int K, int swiglu,
                                                              float glu_limit) {
    extern __shared__ __align__(16) unsigned char gt_smem[];
    bf16* sA = reinterpret_cast<bf16*>(gt_smem);                               // [STAGES][BM][LDS]
    bf16* sW = sA + GT_STAGES * BM * GT_LDS;                                   // [STAGES][BN][LDS]
    __shared__ int s_e, s_first, s_end;
    __shared__ int64_t s_row[BM];
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, e = 0, found = -1;
        for (; e < E; ++e) {
            const int tiles = (offsets[e + 1] - offsets[e] + BM - 1) / BM;
            if (tile < tiles) {
                found = e;
                break;
            }
            tile -= tiles;
        }
        s_e = found;
        if (found >= 0) {
            s_first = offsets[found] + tile * BM;
            s_end = offsets[found + 1];
        }
    }
    __syncthreads();
    const int e = s_e;
    if (e < 0) return;
    const int first = s_first, end = s_end;
    if (threadIdx.x < BM) {
        const int slot = first + threadIdx.x;
        s_row[threadIdx.x] = slot < end ? (a_rows ? (int64_t)a_rows[slot] : (int64_t)slot) : -1;
    }
    __syncthreads();
    const int n0 = blockIdx.x * GT_BN;
    const bf16* We = W + (int64_t)e * N * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int WM = BM >= 64 ? 2 : 1;                 // warps along the slots
    constexpr int WN = 8 / WM;                           // warps along the weight rows
    constexpr int MT = BM / WM / 16;                     // 16-row tiles a warp
    constexpr int NT = GT_BN / WN / 8;                   // 8-column tiles a warp
    const int wm = warp / WN, wn = warp % WN;
    float acc[MT][NT][4] = {};
    const int ktiles = (K + GT_BK - 1) / GT_BK;

    auto load = [&](int kt, int stage) {
        const int k0 = kt * GT_BK;
        bf16* a = sA + stage * BM * GT_LDS;
        bf16* w = sW + stage * GT_BN * GT_LDS;
        for (int i = threadIdx.x; i < BM * (GT_BK / 8); i += 256) {
            const int r = i / (GT_BK / 8), seg = i % (GT_BK / 8);
            const int k = k0 + seg * 8;
            const bool ok = s_row[r] >= 0 && k < K;
            cp_async_16(smem_addr(a + r * GT_LDS + seg * 8), ok ? A + s_row[r] * lda + k : A, ok);
        }
        for (int i = threadIdx.x; i < GT_BN * (GT_BK / 8); i += 256) {
            const int r = i / (GT_BK / 8), seg = i % (GT_BK / 8);
            const int k = k0 + seg * 8, n = n0 + r;
            const bool ok = n < N && k < K;
            cp_async_16(smem_addr(w + r * GT_LDS + seg * 8), ok ? We + (int64_t)n * K + k : We, ok);
        }
    };

#pragma unroll
    for (int st = 0; st < GT_STAGES - 1; ++st) {
        if (st < ktiles) load(st, st);
        cp_async_commit();
    }
    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<GT_STAGES - 2>();
        __syncthreads();
        if (kt + GT_STAGES - 1 < ktiles) load(kt + GT_STAGES - 1, (kt + GT_STAGES - 1) % GT_STAGES);
        cp_async_commit();
        const bf16* a = sA + (kt % GT_STAGES) * BM * GT_LDS;
        const bf16* w = sW + (kt % GT_STAGES) * GT_BN * GT_LDS;
#pragma unroll
        for (int kk = 0; kk < GT_BK; kk += 16) {
            uint32_t af[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int row = wm * (BM / WM) + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(af[mt], smem_addr(a + row * GT_LDS + kk + (lane >> 4) * 8));
            }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t bfr[4];
                const int row = wn * (GT_BN / WN) + np * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(bfr, smem_addr(w + row * GT_LDS + kk + ((lane >> 3) & 1) * 8));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16_16816(acc[mt][2 * np], af[mt], bfr[0], bfr[1]);
                    mma_bf16_16816(acc[mt][2 * np + 1], af[mt], bfr[2], bfr[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int slot = first + wm * (BM / WM) + mt * 16 + g + half * 8;
            if (slot >= end) continue;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int n = n0 + wn * (GT_BN / WN) + nt * 8 + 2 * t;
                const float v0 = acc[mt][nt][half * 2], v1 = acc[mt][nt][half * 2 + 1];
                if (swiglu) {
                    // weight rows 2i and 2i + 1 are the gate and the up row of output i: both are this thread's
                    float g = v0, u = v1, z = v0;
                    if (glu_limit > 0.f) {      // the capped form
                        g = fminf(g, glu_limit);
                        u = fminf(fmaxf(u, -glu_limit), glu_limit) + 1.f;
                        z = 1.702f * g;
                    }
                    if (n + 1 < N) C[(int64_t)slot * ldc + (n >> 1)] = __float2bfloat16_rn(g / (1.f + expf(-z)) * u);
                    continue;
                }
                if (n + 1 < N && (ldc & 1) == 0) {
                    *reinterpret_cast<uint32_t*>(C + (int64_t)slot * ldc + n) = pack_bf16(v0, v1);
                } else {
                    if (n < N) C[(int64_t)slot * ldc + n] = __float2bfloat16_rn(v0);
                    if (n + 1 < N) C[(int64_t)slot * ldc + n + 1] = __float2bfloat16_rn(v1);
                }
            }
        }
    }
}

template <int BM>
static int grouped_gemm_tc_launch(const bf16* A, int64_t lda, const int* a_rows, const bf16* W, bf16* C, int64_t ldc,
                                  const int* offsets, int slots, int E, int N, int K, int swiglu, float glu_limit,
                                  cudaStream_t stream) {
    const int64_t tiles = (slots + BM - 1) / BM + E;
    if (tiles > 65535) return ACORN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)GT_STAGES * (BM + GT_BN) * GT_LDS * sizeof(bf16);
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t err = cudaFuncSetAttribute(grouped_gemm_tc_kernel<BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured.mark();
    }
    dim3 grid((N + GT_BN - 1) / GT_BN, (unsigned)tiles);
    return acorn_launch(grouped_gemm_tc_kernel<BM>, grid, dim3(256), smem, stream, A, lda, a_rows, W, C, ldc, offsets, E, N, K, swiglu, glu_limit);
}

extern "C" int acorn_grouped_gemm_fuses_swiglu(int N, int K, int64_t lda, int dtype) {
    return dtype == ACORN_DTYPE_BF16 && K % 8 == 0 && lda % 8 == 0 && N % 2 == 0;
}

// swiglu: W holds, per output i, the gate row 2i and the up row 2i + 1; C [slots, N / 2] receives
// silu(gate) * up computed from the float32 sums (tensor-core kernel only: see the query above); glu_limit L > 0:
// the capped form min(gate, L) sigmoid(1.702 min(gate, L)) (clamp(up, -L, L) + 1).
extern "C" int acorn_grouped_gemm(const void* A, int64_t lda, const int* a_rows, const void* W, void* C, int64_t ldc,
                                  const int* offsets, int slots, int E, int N, int K, int dtype, int swiglu, float glu_limit,
                                  cudaStream_t stream) {
    if (slots <= 0 || E <= 0 || N <= 0) return 0;
    if (swiglu && !(acorn_grouped_gemm_fuses_swiglu(N, K, lda, dtype) && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0))
        return ACORN_ERR_UNSUPPORTED;
    if (dtype == ACORN_DTYPE_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
        // few rows an expert on average: the small tile (a decode step); else the large one
        if ((int64_t)slots <= (int64_t)16 * E)
            return grouped_gemm_tc_launch<16>((const bf16*)A, lda, a_rows, (const bf16*)W, (bf16*)C, ldc, offsets, slots, E, N, K, swiglu, glu_limit, stream);
        if ((int64_t)slots >= (int64_t)256 * E)          // several full tiles an expert: the tall tile (64 x 32 a warp)
            return grouped_gemm_tc_launch<128>((const bf16*)A, lda, a_rows, (const bf16*)W, (bf16*)C, ldc, offsets, slots, E, N, K, swiglu, glu_limit, stream);
        return grouped_gemm_tc_launch<64>((const bf16*)A, lda, a_rows, (const bf16*)W, (bf16*)C, ldc, offsets, slots, E, N, K, swiglu, glu_limit, stream);
    }
    const int64_t tiles = (slots + GG_BM - 1) / GG_BM + E;       // every expert may end in a partly filled tile
    if (tiles > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid((N + GG_BN - 1) / GG_BN, (unsigned)tiles);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(grouped_gemm_kernel<T>, grid, dim3(256), 0, stream, (const T*)A, lda,
                                                       a_rows, (const T*)W, (T*)C, ldc, offsets, E, N, K));
    return ACORN_ERR_UNSUPPORTED;
}

// out[t, :] = sum over the token's choices, in their order.  With resid32: the float32 sums of the row are
// RMS-normed (x / sqrt(mean(x^2) + eps) * w) and added to resid32[t], and `out` (if given) receives the new
// stream rounded to T: the feed-forward's output norm and residual sum without a kernel of their own.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const T* __restrict__ x, const int* __restrict__ slot_of,
                                   const int* __restrict__ idx, const float* __restrict__ wts, T* __restrict__ out, int H,
                                   int top, int E, float* __restrict__ resid32, const float* __restrict__ norm_w, float eps,
                                   const T* __restrict__ extra) {
    extern __shared__ float row_s[];                    // [H] the row's sums (fused form only)
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int64_t p = t * top + k;
            const float v = idx[p] >= E ? to_float(x[t * H + i]) : to_float(y[(int64_t)slot_of[p] * H + i]);
            acc = fmaf(wts[p], v, acc);
        }
        if (extra) acc += to_float(extra[t * H + i]);      // what every token takes beside its choices (a shared expert)
        if (resid32) {
            row_s[i] = acc;
            ss += acc * acc;
        } else {
            out[t * H + i] = from_float<T>(acc);
        }
    }
    if (!resid32) return;
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = resid32[t * H + i] + row_s[i] * inv * norm_w[i];
        resid32[t * H + i] = v;
        if (out) out[t * H + i] = from_float<T>(v);
    }
}

extern "C" int acorn_moe_combine(const void* y, const void* x, const int* slot_of, const int* idx, const float* wts, void* out,
                                 int tokens, int H, int top, int E, int dtype, float* resid32, const float* norm_w, float eps,
                                 const void* extra, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const size_t smem = resid32 ? (size_t)H * sizeof(float) : 0;
    if (smem > 48 * 1024) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(moe_combine_kernel<T>, dim3(tokens), dim3(256), smem, stream, (const T*)y,
                                                       (const T*)x, slot_of, idx, wts, (T*)out, H, top, E, resid32, norm_w, eps,
                                                       (const T*)extra));
    return ACORN_ERR_UNSUPPORTED;
}
