// Attention through a shared low-rank latent: what happens between the projections and the
// attention kernel, and the per-head matrix products around it.
//
// A token's projection row holds, head by head, [dim unrotated | rot rotated] query entries and, if
// the layer keeps its own cache, rank latent entries followed by rot entries of one rotated key part
// that all heads share.  The cache keeps one row of rank + rot per token: the latent after an RMS
// norm, and the key part after rotation.  With
//     key_h   = [ U_h c | kr ]          (U_h: the head's key up-projection [dim, rank])
//     score_h = (qu_h . U_h c + qr_h . kr) * scale  =  ([U_h^T qu_h | qr_h] . [c | kr]) * scale
// every head attends over the same cached rows with a query of rank + rot entries, and its values are
// V_h (sum_j p_j c_j): one key/value "head" of size rank + rot whose values are the first rank entries
// of the keys.  latent_prep writes the cache row and the rotated query parts; head_linear does the two
// per-head products (U_h^T qu_h before, V_h o_h after the attention).
#include "mma_helpers.cuh"

// ---------------------------------------------------------------- prep
// Rotation: pairs (2i, 2i+1), i < rot_dims / 2, by the angle position * inv_freq[i] (float32); cos and
// sin are multiplied by `mag`.  Entries from rot_dims on pass unchanged.
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int64_t ld, T* __restrict__ qcat,
                                   const float* __restrict__ c_weight, const float* __restrict__ inv_freq, float mag,
                                   const int* __restrict__ positions, const int* __restrict__ token_row,
                                   const int* __restrict__ block_table, const int* __restrict__ page_base,
                                   int table_stride, T* __restrict__ pages, int H, int dim, int rot, int rank,
                                   int rot_dims, int P, float eps, int write_kv, const T* __restrict__ kv_rows,
                                   int64_t ld_kv) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const T* row = proj + (int64_t)t * ld;
    // the rotated query parts, into the tail of every head's query row
    for (int i = threadIdx.x; i < H * rot; i += blockDim.x) {
        const int h = i / rot, e = i % rot;
        const T* src = row + (int64_t)h * (dim + rot) + dim;
        float v;
        if (e < rot_dims) {
            const int pair = e >> 1;
            float s, c;
            sincosf((float)pos * inv_freq[pair], &s, &c);
            s *= mag;
            c *= mag;
            const float a = to_float(src[2 * pair]), b = to_float(src[2 * pair + 1]);
            v = (e & 1) ? (b * c + a * s) : (a * c - b * s);
        } else {
            v = to_float(src[e]);
        }
        qcat[((int64_t)t * H + h) * (rank + rot) + rank + e] = from_float<T>(v);
    }
    if (!write_kv) return;
    // the latent and the shared key part: behind the queries in the same row, or in rows of their own
    const T* kv = kv_rows ? kv_rows + (int64_t)t * ld_kv : row + (int64_t)H * (dim + rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(kv[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)rank + eps);
    const int r = token_row[t];
    const int page = block_table[(int64_t)r * table_stride + pos / P - page_base[r]];
    T* dst = pages + ((int64_t)page * P + pos % P) * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(kv[i]) * inv * c_weight[i]);
    for (int e = threadIdx.x; e < rot; e += blockDim.x) {
        float v;
        if (e < rot_dims) {
            const int pair = e >> 1;
            float s, c;
            sincosf((float)pos * inv_freq[pair], &s, &c);
            s *= mag;
            c *= mag;
            const float a = to_float(kv[rank + 2 * pair]), b = to_float(kv[rank + 2 * pair + 1]);
            v = (e & 1) ? (b * c + a * s) : (a * c - b * s);
        } else {
            v = to_float(kv[rank + e]);
        }
        dst[rank + e] = from_float<T>(v);
    }
}

extern "C" int acorn_latent_prep(const void* proj, int64_t ld, void* qcat, const float* c_weight, const float* inv_freq,
                                 float mag, const int* positions, const int* token_row, const int* block_table,
                                 const int* page_base, int table_stride, void* pages, int tokens, int H, int dim,
                                 int rot, int rank, int rot_dims, int P, float eps, int write_kv, int dtype,
                                 const void* kv_rows, int64_t ld_kv, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot || rot < 0 || rank < 1 || P < 1) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(latent_prep_kernel<T>, dim3(tokens), dim3(128), 0, stream,
                                                       (const T*)proj, ld, (T*)qcat, c_weight, inv_freq, mag, positions,
                                                       token_row, block_table, page_base, table_stride, (T*)pages, H,
                                                       dim, rot, rank, rot_dims, P, eps, write_kv, (const T*)kv_rows, ld_kv));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- per-head matrix products
// y[t, h, o] = sum_i w[h, o, i] * x[t, h, i]: x and y with a token stride and a head stride each (in
// elements; the innermost dimension contiguous), w [H, O, I] contiguous.  float32 accumulation, one
// chain over i = 0, 1, ... per output, so a token's result does not depend on the other tokens.
#define HL_TM 16
#define HL_TN 64
#define HL_TK 32

template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, int64_t xs_t, int64_t xs_h,
                                                          const T* __restrict__ w, T* __restrict__ y, int64_t ys_t,
                                                          int64_t ys_h, int tokens, int O, int I) {
    __shared__ float xs[HL_TM][HL_TK + 1];
    __shared__ float ws[HL_TN][HL_TK + 1];
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.z;
    const int t0 = blockIdx.x * HL_TM, o0 = blockIdx.y * HL_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 output groups of 4, 16 tokens
    const T* wh = w + (int64_t)h * O * I;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < I; k0 += HL_TK) {
        for (int e = threadIdx.x; e < HL_TM * HL_TK; e += 256) {
            const int tt = e / HL_TK, kk = e % HL_TK;
            const int t = t0 + tt, k = k0 + kk;
            xs[tt][kk] = (t < tokens && k < I) ? to_float(x[(int64_t)t * xs_t + (int64_t)h * xs_h + k]) : 0.f;
        }
        for (int e = threadIdx.x; e < HL_TN * HL_TK; e += 256) {
            const int oo = e / HL_TK, kk = e % HL_TK;
            const int o = o0 + oo, k = k0 + kk;
            ws[oo][kk] = (o < O && k < I) ? to_float(wh[(int64_t)o * I + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HL_TK; ++kk) {
            const float a = xs[ty][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(a, ws[tx + 16 * j][kk], acc[j]);
        }
        __syncthreads();
    }
    const int t = t0 + ty;
    if (t < tokens) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o < O) y[(int64_t)t * ys_t + (int64_t)h * ys_h + o] = from_float<T>(acc[j]);
        }
    }
}

// The same for few tokens (a decode step): a block takes a head, up to HLR_TM tokens (their x rows wait in shared
// memory as float32) and a run of outputs; a warp takes an output at a time, its lanes four weights each per 128
// inputs (8- or 16-byte reads), and reduces the tokens' partial sums by shuffles.  A token's chain of sums is fixed
// by the lane partition, so its result does not depend on the other tokens here either.
#define HLR_TM 8
template <typename T>
__global__ void __launch_bounds__(256) head_linear_rows_kernel(const T* __restrict__ x, int64_t xs_t, int64_t xs_h,
                                                               const T* __restrict__ w, T* __restrict__ y, int64_t ys_t,
                                                               int64_t ys_h, int tokens, int O, int I, int rows_per_block) {
    extern __shared__ __align__(16) float hlr_x[];                 // [HLR_TM][I]
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.y, t0 = blockIdx.z * HLR_TM;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < HLR_TM * I; e += 256) {
        const int tt = e / I, i = e - tt * I;
        hlr_x[e] = (t0 + tt < tokens) ? to_float(x[(int64_t)(t0 + tt) * xs_t + (int64_t)h * xs_h + i]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (int64_t)h * O * I;
    const int o_end = min(O, (int)(blockIdx.x + 1) * rows_per_block);
    for (int o = blockIdx.x * rows_per_block + warp; o < o_end; o += 8) {
        const T* wr = wh + (int64_t)o * I;
        float acc[HLR_TM];
#pragma unroll
        for (int t = 0; t < HLR_TM; ++t) acc[t] = 0.f;
        for (int i0 = lane * 4; i0 < I; i0 += 128) {
            const float4 wv = Vec4<T>::load(wr + i0);
#pragma unroll
            for (int t = 0; t < HLR_TM; ++t) {
                const float4 a = *reinterpret_cast<const float4*>(hlr_x + t * I + i0);
                acc[t] = fmaf(wv.x, a.x, fmaf(wv.y, a.y, fmaf(wv.z, a.z, fmaf(wv.w, a.w, acc[t]))));
            }
        }
        float mine = 0.f;
#pragma unroll
        for (int t = 0; t < HLR_TM; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == t) mine = v;
        }
        if (lane < HLR_TM && t0 + lane < tokens) y[(int64_t)(t0 + lane) * ys_t + (int64_t)h * ys_h + o] = from_float<T>(mine);
    }
}
#define HLR_MAX_TOKENS 32

extern "C" int acorn_head_linear(const void* x, int64_t xs_t, int64_t xs_h, const void* w, void* y, int64_t ys_t,
                                 int64_t ys_h, int tokens, int H, int O, int I, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || H <= 0 || O <= 0) return 0;
    if (tokens <= HLR_MAX_TOKENS && I % 4 == 0 && (size_t)HLR_TM * I * sizeof(float) <= 48 * 1024 && H <= 65535) {
        const int rpb = (int64_t)H * ((O + 7) / 8) >= 592 ? 16 : 8;
        dim3 grid((O + rpb - 1) / rpb, H, (tokens + HLR_TM - 1) / HLR_TM);
        const size_t smem = (size_t)HLR_TM * I * sizeof(float);
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(head_linear_rows_kernel<T>, grid, dim3(256), smem, stream, (const T*)x,
                                                           xs_t, xs_h, (const T*)w, (T*)y, ys_t, ys_h, tokens, O, I, rpb));
    }
    if (H > 65535 || (O + HL_TN - 1) / HL_TN > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid((tokens + HL_TM - 1) / HL_TM, (O + HL_TN - 1) / HL_TN, H);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(head_linear_kernel<T>, grid, dim3(256), 0, stream, (const T*)x, xs_t,
                                                       xs_h, (const T*)w, (T*)y, ys_t, ys_h, tokens, O, I));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- attention over the cached rows, tensor cores
// bfloat16.  All heads of a token attend over the same cached rows, so the (token, head) pairs of a few
// neighbouring tokens are the rows of one matrix: a block takes LA_M = 64 of them (64 / H tokens of one
// request, listed on the host as tiles (row, first token)), which are 64 consecutive rows of q [T, H, d]
// and of the output [T, H, dv].  Keys come in blocks of 64 through shared memory (cp.async, two buffers
// where they fit).  Eight warps.  Scores: warp (rg, kh) multiplies 16 rows by 32 keys over d (mma.sync
// m16n8k16); the row maxima of the two key halves meet in shared memory; the weights (float32, exp of
// the float32 scores) go to shared memory as bfloat16, the operand of the second product.  Values: the
// first dv entries of the same key rows; warp (rh, cq) owns 32 rows by a quarter of the dv columns of the
// float32 accumulator.  Window: query at position p sees keys p - window + 1 .. p.  Sink: exp(sink_h) is
// added to a row's denominator at the end.  With few tiles (a decode step) the key blocks of a tile are
// shared out over `splits` blocks, which leave unnormalized sums, maxima and denominators for a merge kernel.
#define LA_M 64
#define LA_KB 64
#define LA_THREADS 256
#define LA_PLD 72

template <int NT>
__global__ void __launch_bounds__(LA_THREADS) latent_attention_tc_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ pages, const int* __restrict__ block_table,
    const int* __restrict__ page_base, int table_stride, const int* __restrict__ row_start, const int* __restrict__ row_pos,
    const int* __restrict__ tiles, const float* __restrict__ sink, float scale, int window, int H, int d, int dv, int logP,
    int kbufs, int splits, float* __restrict__ part) {
    extern __shared__ __align__(16) unsigned char la_smem[];
    const int lds = d + 8;
    bf16* Qs = reinterpret_cast<bf16*>(la_smem);                 // [64][lds]
    bf16* Ks = Qs + LA_M * lds;                                  // [kbufs][64][lds]
    bf16* Ps = Ks + (size_t)kbufs * LA_KB * lds;                 // [64][72]
    float* red = reinterpret_cast<float*>(Ps + LA_M * LA_PLD);   // [2][64]: maxima, at the end sums, of the key halves
    float* corr_s = red + 2 * LA_M;                              // [64]
    pdl_wait();
    pdl_trigger();
    const int r = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
    const int first = row_start[r], len = row_start[r + 1] - first;
    const int TQ = LA_M / H;
    const int ntok = min(TQ, len - q0), rows_valid = ntok * H;
    const int p_first = row_pos[r] + q0, p_last = p_first + ntok - 1;
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int* table = block_table + (int64_t)r * table_stride - page_base[r];
    const int pmask = (1 << logP) - 1;
    const int segs = d / 8;
    const int64_t qrow0 = (int64_t)(first + q0) * H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3, mat = lane >> 3, rr = lane & 7;

    for (int idx = threadIdx.x; idx < LA_M * segs; idx += LA_THREADS) {
        const int row = idx / segs, seg = idx - row * segs;
        const bool ok = row < rows_valid;
        cp_async_16(smem_addr(Qs + row * lds + seg * 8), ok ? q + (qrow0 + row) * d + seg * 8 : q, ok);
    }
    auto load_keys = [&](int kb, int buf) {
        bf16* dst = Ks + (size_t)buf * LA_KB * lds;
        for (int idx = threadIdx.x; idx < LA_KB * segs; idx += LA_THREADS) {
            const int row = idx / segs, seg = idx - row * segs;
            const int key = kb + row;
            const bool ok = key >= key_lo && key <= p_last;
            const bf16* src = pages;
            if (ok) src = pages + ((((int64_t)__ldg(table + (key >> logP))) << logP) + (key & pmask)) * d + seg * 8;
            cp_async_16(smem_addr(dst + row * lds + seg * 8), src, ok);
        }
    };
    const int kb_first = (key_lo / LA_KB) * LA_KB;
    const int nblk = (p_last - kb_first) / LA_KB + 1;
    // with splits (blockIdx.y), a block takes a contiguous share of the key blocks and leaves partial results
    const int per = (nblk + splits - 1) / splits;
    const int it0 = min(nblk, (int)blockIdx.y * per), it1 = min(nblk, it0 + per);
    if (it0 < it1) load_keys(kb_first + it0 * LA_KB, 0);
    cp_async_commit();

    // score phase: rows rg*16 + g and + 8, keys kh*32 ..
    const int rg = warp & 3, kh = warp >> 2;
    const int row_a = rg * 16 + g, row_b = row_a + 8;
    const bool valid_a = row_a < rows_valid, valid_b = row_b < rows_valid;
    const int p_a = p_first + row_a / H, p_b = p_first + row_b / H;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // value phase: rows rh*32 .., columns cq * NT * 8 ..
    const int rh = warp >> 2, cq = warp & 3;
    const int colbase = cq * NT * 8;
    float o[2][NT][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) o[mt][nt][c] = 0.f;

    for (int it = it0; it < it1; ++it) {
        const int kb = kb_first + it * LA_KB;
        const int buf = kbufs == 2 ? ((it - it0) & 1) : 0;
        if (kbufs == 2 && it + 1 < it1) load_keys(kb + LA_KB, (it + 1 - it0) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                         // this block's keys (and the queries) are here
        const bf16* ks_ = Ks + (size_t)buf * LA_KB * lds;
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) sc[nt][c] = 0.f;
        for (int k0 = 0; k0 < d; k0 += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_addr(Qs + (rg * 16 + rr + (mat & 1) * 8) * lds + k0 + (mat >> 1) * 8));
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_addr(ks_ + (kh * 32 + j2 * 16 + (mat >> 1) * 8 + rr) * lds + k0 + (mat & 1) * 8));
                mma_bf16_16816(sc[2 * j2], a, b[0], b[1]);
                mma_bf16_16816(sc[2 * j2 + 1], a, b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = kb + kh * 32 + nt * 8 + 2 * t + (c & 1);
                const int hh = c >> 1;
                const int pos = hh ? p_b : p_a;
                const bool ok = (hh ? valid_b : valid_a) && key <= pos && (window <= 0 || key > pos - window);
                sc[nt][c] = ok ? sc[nt][c] * scale : -INFINITY;
                mx[hh] = fmaxf(mx[hh], sc[nt][c]);
            }
        }
        mx[0] = quad_max(mx[0]);
        mx[1] = quad_max(mx[1]);
        if (t == 0) {
            red[kh * LA_M + row_a] = mx[0];
            red[kh * LA_M + row_b] = mx[1];
        }
        __syncthreads();                                         // the maxima of both key halves
        float msafe[2], corr[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int row = hh ? row_b : row_a;
            const float m_new = fmaxf(m[hh], fmaxf(red[row], red[LA_M + row]));
            msafe[hh] = m_new == -INFINITY ? 0.f : m_new;
            corr[hh] = expf(m[hh] - msafe[hh]);                  // nothing seen before: exp(-inf) = 0
            m[hh] = m_new;
        }
        float ps[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float e0 = expf(sc[nt][0] - msafe[0]), e1 = expf(sc[nt][1] - msafe[0]);
            const float e2 = expf(sc[nt][2] - msafe[1]), e3 = expf(sc[nt][3] - msafe[1]);
            ps[0] += e0 + e1;
            ps[1] += e2 + e3;
            const int col = kh * 32 + nt * 8 + 2 * t;
            *reinterpret_cast<uint32_t*>(Ps + row_a * LA_PLD + col) = pack_bf16(e0, e1);
            *reinterpret_cast<uint32_t*>(Ps + row_b * LA_PLD + col) = pack_bf16(e2, e3);
        }
        l[0] = l[0] * corr[0] + ps[0];
        l[1] = l[1] * corr[1] + ps[1];
        if (kh == 0 && t == 0) {
            corr_s[row_a] = corr[0];
            corr_s[row_b] = corr[1];
        }
        __syncthreads();                                         // the weights and the rows' corrections
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const float ca = corr_s[rh * 32 + mt * 16 + g], cb = corr_s[rh * 32 + mt * 16 + g + 8];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                o[mt][nt][0] *= ca;
                o[mt][nt][1] *= ca;
                o[mt][nt][2] *= cb;
                o[mt][nt][3] *= cb;
            }
        }
#pragma unroll
        for (int kk = 0; kk < LA_KB / 16; ++kk) {
            uint32_t pa[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
                ldmatrix_x4(pa[mt], smem_addr(Ps + (rh * 32 + mt * 16 + rr + (mat & 1) * 8) * LA_PLD + kk * 16 + (mat >> 1) * 8));
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                const int col = colbase + n2 * 16;
                if (col < dv) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_addr(ks_ + (kk * 16 + (mat & 1) * 8 + rr) * lds + col + (mat >> 1) * 8));
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma_bf16_16816(o[mt][2 * n2], pa[mt], b[0], b[1]);
                        mma_bf16_16816(o[mt][2 * n2 + 1], pa[mt], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                         // the keys' buffer, the weights and the maxima are free
        if (kbufs == 1 && it + 1 < it1) {
            load_keys(kb + LA_KB, 0);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    // the rows' denominators: the two key halves' sums, and the sink
    l[0] = quad_sum(l[0]);
    l[1] = quad_sum(l[1]);
    if (t == 0) {
        red[kh * LA_M + row_a] = l[0];
        red[kh * LA_M + row_b] = l[1];
        if (kh == 0) {
            corr_s[row_a] = m[0];
            corr_s[row_b] = m[1];
        }
    }
    __syncthreads();
    if (splits > 1) {
        // partial results of this share of the keys: the unnormalized sums, then the row's maximum and denominator
        float* mine = part + ((int64_t)blockIdx.x * splits + blockIdx.y) * LA_M * (dv + 2);
        if (threadIdx.x < LA_M) {
            mine[(int64_t)threadIdx.x * (dv + 2) + dv] = corr_s[threadIdx.x];
            mine[(int64_t)threadIdx.x * (dv + 2) + dv + 1] = red[threadIdx.x] + red[LA_M + threadIdx.x];
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int row = rh * 32 + mt * 16 + g + hh * 8;
                if (row >= rows_valid) continue;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int col = colbase + nt * 8 + 2 * t;
                    if (col < dv) {
                        mine[(int64_t)row * (dv + 2) + col] = o[mt][nt][hh * 2];
                        mine[(int64_t)row * (dv + 2) + col + 1] = o[mt][nt][hh * 2 + 1];
                    }
                }
            }
        return;
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int row = rh * 32 + mt * 16 + g + hh * 8;
            if (row >= rows_valid) continue;
            float total = red[row] + red[LA_M + row];
            if (sink) total += expf(sink[row % H] - corr_s[row]);
            const float inv = 1.f / total;
            bf16* dst = out + (qrow0 + row) * dv;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = colbase + nt * 8 + 2 * t;
                if (col < dv)
                    *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[mt][nt][hh * 2] * inv, o[mt][nt][hh * 2 + 1] * inv);
            }
        }
    }
}

// One block per (tile, row): the shares' partial results, weighted by exp(their maximum - the common one), over
// the sum of their denominators and the sink's term.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part, bf16* __restrict__ out,
                                              const int* __restrict__ row_start, const int* __restrict__ tiles,
                                              const float* __restrict__ sink, int H, int dv, int splits) {
    pdl_wait();
    pdl_trigger();
    const int tile = blockIdx.x, row = blockIdx.y;
    const int r = tiles[2 * tile], q0 = tiles[2 * tile + 1];
    const int first = row_start[r], len = row_start[r + 1] - first;
    const int ntok = min(LA_M / H, len - q0);
    if (row >= ntok * H) return;
    const float* base = part + (int64_t)tile * splits * LA_M * (dv + 2) + (int64_t)row * (dv + 2);
    const int64_t stride = (int64_t)LA_M * (dv + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, base[s * stride + dv]);
    float total = sink ? expf(sink[row % H] - m) : 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = base[s * stride + dv];
        if (ms > -INFINITY) total += base[s * stride + dv + 1] * expf(ms - m);
    }
    const float inv = 1.f / total;
    bf16* dst = out + ((int64_t)(first + q0) * H + row) * dv;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = base[s * stride + dv];
            if (ms > -INFINITY) acc += base[s * stride + c] * expf(ms - m);
        }
        dst[c] = __float2bfloat16_rn(acc * inv);
    }
}

static size_t latent_tc_smem(int d, int kbufs) {
    return (size_t)(LA_M + kbufs * LA_KB) * (d + 8) * sizeof(bf16) + (size_t)LA_M * LA_PLD * sizeof(bf16) + 3 * LA_M * sizeof(float);
}

extern "C" int acorn_latent_attention_tc_supported(int H, int d, int dv, int P) {
    return H >= 1 && H <= LA_M && d % 16 == 0 && dv % 16 == 0 && dv >= 16 && dv <= d && dv <= 512 && acorn_log2_exact(P) >= 0 &&
           latent_tc_smem(d, 1) <= 220 * 1024;
}

template <int NT>
static int latent_tc_launch(const bf16* q, bf16* out, const bf16* pages, const int* block_table, const int* page_base,
                            int table_stride, const int* row_start, const int* row_pos, const int* tiles, int num_tiles,
                            const float* sink, float scale, int window, int H, int d, int dv, int logP, int splits, float* part,
                            cudaStream_t stream) {
    const int kbufs = latent_tc_smem(d, 2) <= 220 * 1024 ? 2 : 1;
    static AcornPerDevice configured;
    if (!configured.seen()) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured.mark();
    }
    int rc = acorn_launch(latent_attention_tc_kernel<NT>, dim3(num_tiles, splits), dim3(LA_THREADS), latent_tc_smem(d, kbufs), stream,
                          q, out, pages, block_table, page_base, table_stride, row_start, row_pos, tiles, sink, scale, window, H, d,
                          dv, logP, kbufs, splits, part);
    if (rc != 0 || splits == 1) return rc;
    return acorn_launch(latent_attention_merge_kernel, dim3(num_tiles, LA_M), dim3(128), 0, stream, (const float*)part, out, row_start,
                        tiles, sink, H, dv, splits);
}

extern "C" int acorn_latent_attention_tc(const void* q, void* out, const void* pages, const int* block_table, const int* page_base,
                                         int table_stride, const int* row_start, const int* row_pos, const int* tiles,
                                         int num_tiles, const float* sink, float scale, int window, int H, int d, int dv, int P,
                                         int splits, float* part, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (!acorn_latent_attention_tc_supported(H, d, dv, P)) return ACORN_ERR_UNSUPPORTED;
    if (splits < 1 || splits > 65535 || (splits > 1 && part == nullptr)) return ACORN_ERR_UNSUPPORTED;
    const int logP = acorn_log2_exact(P);
#define LA_ARGS (const bf16*)q, (bf16*)out, (const bf16*)pages, block_table, page_base, table_stride, row_start, row_pos, tiles, \
                num_tiles, sink, scale, window, H, d, dv, logP, splits, part, stream
    if (dv <= 64) return latent_tc_launch<2>(LA_ARGS);
    if (dv <= 128) return latent_tc_launch<4>(LA_ARGS);
    if (dv <= 256) return latent_tc_launch<8>(LA_ARGS);
    if (dv <= 384) return latent_tc_launch<12>(LA_ARGS);
    return latent_tc_launch<16>(LA_ARGS);
#undef LA_ARGS
}
