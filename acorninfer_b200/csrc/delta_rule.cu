// Gated delta rule with one decay per key channel, as a recurrent mixer's kernels.
//
// Per head a state matrix S [dim, vdim] in float32, zero when a request starts, kept in the
// request's state slot between steps.  For every token, with unit-length q and k (q times dim^-1/2),
// a write strength beta and a decay g[d] per key channel, all float32:
//     S[d, :] *= g[d];   u = beta * (v - S^T k);   S += k u^T;   o = S^T q.
// The columns of S (one per value channel) never mix, so a block takes a head's columns in tiles.
//
//   delta_prep          per token: the short causal convolution over time of the q, k, v channels
//                       (inputs before the step's first token come from the request's state), silu,
//                       unit norms, beta = sigmoid(.), g = exp(-exp(A_log) softplus(. + dt_bias)),
//                       the output gate sigmoid(.); float32 outputs
//   conv_state_update   per row: the last taps - 1 convolution inputs into the request's state
//   delta_rule          the recurrence over a row's tokens, state in registers
//   delta_out           per token and head: o / rms(o) * w * gate
//
// The state slot is one float32 vector: S of all heads [H, dim, vdim], then the convolution inputs
// [taps - 1, channels] in time order.
#include "common.cuh"

#define DELTA_MAX_TAPS 16

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// main [T, C + H]: the q (KH*dim), k (KH*dim), v (H*vdim) channels before the convolution, then beta's
// pre-activation per head.  up [T, H*dim + H*vdim] float32: the decay's and the gate's pre-activations.
template <typename T>
__global__ void delta_prep_kernel(const T* __restrict__ main_, int64_t ld, const float* __restrict__ up, int64_t ld_up,
                                  const float* __restrict__ conv_w, const float* __restrict__ state, int64_t slot_stride,
                                  int64_t conv_off, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                  const int* __restrict__ token_row, const int* __restrict__ row_start,
                                  const int* __restrict__ row_slot, float* __restrict__ qn, float* __restrict__ kn,
                                  float* __restrict__ vv, float* __restrict__ beta, float* __restrict__ g,
                                  float* __restrict__ gate, int H, int KH, int dim, int vdim, int taps) {
    extern __shared__ float act[];                      // [C] activations of the q, k, v channels
    __shared__ float inv_norm[2 * 64];                  // per q head, per k head (KH <= 64)
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int r = token_row[t];
    const int i0 = t - row_start[r];                    // index of the token within its row
    const int C = 2 * KH * dim + H * vdim;
    const float* cstate = state + (int64_t)row_slot[r] * slot_stride + conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int idx = i0 - (taps - 1) + j;        // input index within the row; negative: before the step
            const float in = idx >= 0 ? to_float(main_[(int64_t)(t - i0 + idx) * ld + c])
                                      : cstate[(int64_t)(taps - 1 + idx) * C + c];
            acc = fmaf(conv_w[(int64_t)c * taps + j], in, acc);
        }
        act[c] = acc * sigmoidf_(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int hd = warp; hd < 2 * KH; hd += nwarps) {    // unit norms of the q heads, then of the k heads
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) ss += act[hd * dim + d] * act[hd * dim + d];
        ss = warp_sum(ss);
        if (lane == 0) inv_norm[hd] = rsqrtf(ss + 1e-6f);
    }
    __syncthreads();
    const float qscale = rsqrtf((float)dim);
    for (int c = threadIdx.x; c < KH * dim; c += blockDim.x) {
        qn[(int64_t)t * KH * dim + c] = act[c] * inv_norm[c / dim] * qscale;
        kn[(int64_t)t * KH * dim + c] = act[KH * dim + c] * inv_norm[KH + c / dim];
    }
    for (int c = threadIdx.x; c < H * vdim; c += blockDim.x) {
        vv[(int64_t)t * H * vdim + c] = act[2 * KH * dim + c];
        gate[(int64_t)t * H * vdim + c] = sigmoidf_(up[(int64_t)t * ld_up + H * dim + c]);
    }
    for (int c = threadIdx.x; c < H * dim; c += blockDim.x)
        g[(int64_t)t * H * dim + c] = expf(-expf(A_log[c / dim]) * softplusf_(up[(int64_t)t * ld_up + c] + dt_bias[c]));
    for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(int64_t)t * H + h] = sigmoidf_(to_float(main_[(int64_t)t * ld + C + h]));
}

extern "C" int acorn_delta_prep(const void* main_, int64_t ld, const float* up, int64_t ld_up, const float* conv_w,
                                const float* state, int64_t slot_stride, int64_t conv_off, const float* A_log,
                                const float* dt_bias, const int* token_row, const int* row_start, const int* row_slot,
                                float* qn, float* kn, float* vv, float* beta, float* g, float* gate, int tokens, int H,
                                int KH, int dim, int vdim, int taps, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int64_t C = 2 * (int64_t)KH * dim + (int64_t)H * vdim;
    if (KH < 1 || KH > 64 || H % KH || taps < 1 || taps > DELTA_MAX_TAPS || C * 4 > 160 * 1024) return ACORN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 48 * 1024) {
        static AcornPerDevice configured;
        if (!configured.seen()) {
            cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(delta_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return (int)e;
            configured.mark();
        }
    }
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(delta_prep_kernel<T>, dim3(tokens), dim3(256), smem, stream,
                                                       (const T*)main_, ld, up, ld_up, conv_w, state, slot_stride, conv_off,
                                                       A_log, dt_bias, token_row, row_start, row_slot, qn, kn, vv, beta, g,
                                                       gate, H, KH, dim, vdim, taps));
    return ACORN_ERR_UNSUPPORTED;
}

// The convolution's memory after the step: the last taps - 1 inputs of the request, i.e. of the old
// memory followed by the row's inputs (plus a bias per channel, if one is given).  A thread owns a channel of a row, reads what it needs and
// only then writes, so a row shorter than the memory shifts it correctly.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ main_, int64_t ld, float* __restrict__ state,
                                         int64_t slot_stride, int64_t conv_off, const int* __restrict__ row_start,
                                         const int* __restrict__ row_slot, int C, int taps, int skip_single,
                                         const float* __restrict__ bias) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = row_start[r], L = row_start[r + 1] - first;
    if (skip_single && L == 1) return;                  // the kernel before this one has shifted the memory of such rows
    float* cs = state + (int64_t)row_slot[r] * slot_stride + conv_off;
    float keep[DELTA_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < DELTA_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int idx = L + j - (taps - 1);         // index into the row's inputs; negative: old memory
            keep[j] = idx >= 0 ? to_float(main_[(int64_t)(first + idx) * ld + c]) + (bias ? bias[c] : 0.f)
                               : cs[(int64_t)(L + j) * C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < DELTA_MAX_TAPS - 1; ++j)
        if (j < taps - 1) cs[(int64_t)j * C + c] = keep[j];
}

extern "C" int acorn_conv_state_update(const void* main_, int64_t ld, float* state, int64_t slot_stride, int64_t conv_off,
                                       const int* row_start, const int* row_slot, int rows, int C, int taps, int dtype,
                                       int skip_single, const float* bias, cudaStream_t stream) {
    if (rows <= 0 || taps <= 1) return 0;
    if (taps > DELTA_MAX_TAPS || rows > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid((C + 127) / 128, rows);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(conv_state_update_kernel<T>, grid, dim3(128), 0, stream,
                                                       (const T*)main_, ld, state, slot_stride, conv_off, row_start,
                                                       row_slot, C, taps, skip_single, bias));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- the recurrence
// A block: one row, one head, 32 value channels.  Thread (column, slice): the state entries S[d, column]
// for d = slice, slice + 4, ... (DPT of them, in registers).  The four slices of a column sit in
// neighbouring lanes and add their partial dot products by two shuffles.
//
// What a token needs of S is one pass: with gk = g * k and gq = g * q (per key channel),
//     a = sum_d S[d] gk[d]   (= (g S)^T k),      b = sum_d S[d] gq[d]   (= (g S)^T q),
//     u = beta (v - a),      o = b + (k . q) u,    S[d] = g[d] S[d] + k[d] u,
// so the two sums are reduced together and nothing is reduced after the update: the update of one
// token overlaps the sums of the next.  The tokens' q, k, g, v, beta come through shared memory, `stage`
// tokens at a time: the next stage's rows are fetched (cp.async) while this one is computed; gk, gq, g, k
// are packed per channel into one 16-byte entry, and k . q is summed, once per stage.
#define DELTA_THREADS 256

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

//
// PRE (a recurrence without the delta correction whose output reads the state before the token's decay and
// write, and sees the token itself through a bonus u per head and key channel: time mixing of the RWKV kind):
//     o = S^T q + (sum_d q[d] u[d] k[d]) v,      S[d] = g[d] S[d] + k[d] v.
// It is the same loop with gq = q, no sum against gk, beta = 1 and the bonus inside the k . q sum.
//
// In that form the state moves by S <- diag(g) S + k v^T, so a long row can be cut into segments that run side
// by side (a recurrence is sequential over a row's tokens, and a prompt alone in its step would otherwise keep
// a few dozen blocks busy): pass 1 runs every segment from a zero state to its end state E_j and multiplies up its
// decays P_j; delta_fold walks the segments, S_j = diag(P_(j-1)) S_(j-1) + E_(j-1), leaving each segment's true
// start state in the scratch and the row's end state in the request's slot; pass 2 runs every segment again from
// its start state and writes the outputs.
struct DeltaSegments {
    int pass;                 // 0: rows in one piece; 1, 2: the passes above
    int nseg, seg_len;        // segments a row, tokens a segment
    float* seg_state;         // [rows * nseg, H, dim, vdim]
    float* seg_decay;         // [rows * nseg, H, dim]
};
// CPT: columns a thread holds (an entry read from shared memory then serves them all); NT: threads a block.
template <int DPT, int DELTA_SLICES, bool PRE, int CPT, int NT>
__global__ void __launch_bounds__(NT) delta_rule_kernel(
    const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
    const float* __restrict__ beta, const float* __restrict__ g, float* __restrict__ state, int64_t slot_stride,
    const int* __restrict__ row_start, const int* __restrict__ row_slot, float* __restrict__ out, int H, int KH, int dim,
    int vdim, int stage, const float* __restrict__ bonus, DeltaSegments sg) {
    constexpr int DELTA_COLS = NT / DELTA_SLICES * CPT;                // value channels a block
    extern __shared__ __align__(16) float sm[];
    constexpr int DIMP = DPT * DELTA_SLICES;                           // dim rounded up: entries beyond dim are zero
    float4* pack = reinterpret_cast<float4*>(sm);                      // [stage][DIMP]: gk, gq, g, k
    float* raw = sm + (size_t)stage * DIMP * 4;                        // [2][stage][3][dim] q, k, g as fetched
    float* sv = raw + (size_t)2 * stage * 3 * dim;                     // [2][stage][COLS]
    float* sb = sv + 2 * stage * DELTA_COLS;                           // [2][stage]
    float* skq = sb + 2 * stage;                                       // [stage]
    pdl_wait();
    pdl_trigger();
    const int r = sg.pass ? blockIdx.x / sg.nseg : blockIdx.x, seg = sg.pass ? blockIdx.x % sg.nseg : 0;
    const int h = blockIdx.y, c0 = blockIdx.z * DELTA_COLS;
    const int kh = h / (H / KH);
    const int slice = threadIdx.x & (DELTA_SLICES - 1), col = threadIdx.x / DELTA_SLICES;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int column = c0 + col * CPT;                                 // the first of this thread's columns
    bool live[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) live[j] = column + j < vdim;
    float* S_g = sg.pass ? sg.seg_state + (((int64_t)r * sg.nseg + seg) * H + h) * dim * vdim
                         : state + (int64_t)row_slot[r] * slot_stride + (int64_t)h * dim * vdim;
    float S[CPT][DPT], Pd[DPT];                                        // Pd: the segment's decays multiplied up (pass 1)
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = slice + DELTA_SLICES * i;
#pragma unroll
        for (int j = 0; j < CPT; ++j) S[j][i] = (sg.pass != 1 && live[j] && d < dim) ? S_g[(int64_t)d * vdim + column + j] : 0.f;
        Pd[i] = 1.f;
    }
    int first = row_start[r], last = row_start[r + 1];
    if (sg.pass) {
        first = min(last, first + seg * sg.seg_len);
        last = min(last, first + sg.seg_len);
    }
    const int stages = (last - first + stage - 1) / stage;

    auto fetch = [&](int s) {
        const int t0 = first + s * stage, n = min(stage, last - t0);
        float* rw = raw + (size_t)(s & 1) * stage * 3 * dim;
        for (int e = threadIdx.x; e < n * dim; e += blockDim.x) {
            const int tt = e / dim, d = e - tt * dim;
            const int64_t t = t0 + tt;
            cp_async_4(rw + (tt * 3 + 0) * dim + d, qn + (t * KH + kh) * dim + d);
            cp_async_4(rw + (tt * 3 + 1) * dim + d, kn + (t * KH + kh) * dim + d);
            cp_async_4(rw + (tt * 3 + 2) * dim + d, g + (t * H + h) * dim + d);
        }
        for (int e = threadIdx.x; e < n * DELTA_COLS; e += blockDim.x) {
            const int tt = e / DELTA_COLS, cc = e % DELTA_COLS;
            float* dst = sv + ((s & 1) * stage + tt) * DELTA_COLS + cc;
            if (c0 + cc < vdim) cp_async_4(dst, vv + ((int64_t)(t0 + tt) * H + h) * vdim + c0 + cc);
            else *dst = 0.f;
        }
        if (!PRE && threadIdx.x < n) cp_async_4(sb + (s & 1) * stage + threadIdx.x, beta + (int64_t)(t0 + threadIdx.x) * H + h);
    };

    if (stages > 0) fetch(0);
    asm volatile("cp.async.commit_group;\n" ::);
    for (int s = 0; s < stages; ++s) {
        if (s + 1 < stages) fetch(s + 1);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();                                               // stage s has arrived
        const int t0 = first + s * stage, n = min(stage, last - t0);
        const float* rw = raw + (size_t)(s & 1) * stage * 3 * dim;
        for (int e = threadIdx.x; e < n * DIMP; e += blockDim.x) {
            const int tt = e / DIMP, d = e % DIMP;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (d < dim) {
                const float q = rw[(tt * 3 + 0) * dim + d], k = rw[(tt * 3 + 1) * dim + d], gg = rw[(tt * 3 + 2) * dim + d];
                v = PRE ? make_float4(0.f, q, gg, k) : make_float4(gg * k, gg * q, gg, k);
            }
            pack[e] = v;
        }
        for (int tt = warp; tt < n; tt += NT / 32) {
            float kq = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float qd = PRE ? rw[(tt * 3 + 0) * dim + d] * bonus[(int64_t)h * dim + d] : rw[(tt * 3 + 0) * dim + d];
                kq = fmaf(qd, rw[(tt * 3 + 1) * dim + d], kq);
            }
            kq = warp_sum(kq);
            if (lane == 0) skq[tt] = kq;
        }
        __syncthreads();
        const float* v_s = sv + (s & 1) * stage * DELTA_COLS;
        const float* b_s = sb + (s & 1) * stage;
#pragma unroll 4
        for (int tt = 0; tt < n; ++tt) {
            const float4* p = pack + tt * DIMP + slice;                // this thread's channels: every SLICES-th entry
            float4 e[DPT];
#pragma unroll
            for (int i = 0; i < DPT; ++i) e[i] = p[DELTA_SLICES * i];
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                float a = 0.f, b = 0.f;
                if (!PRE || sg.pass != 1) {                            // a segment's first pass writes no output
                    float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                    for (int i = 0; i < DPT; i += 2) {
                        if (!PRE) a0 = fmaf(S[j][i], e[i].x, a0);
                        b0 = fmaf(S[j][i], e[i].y, b0);
                        if (!PRE) a1 = fmaf(S[j][i + 1], e[i + 1].x, a1);
                        b1 = fmaf(S[j][i + 1], e[i + 1].y, b1);
                    }
                    a = a0 + a1;
                    b = b0 + b1;
#pragma unroll
                    for (int o = 1; o < DELTA_SLICES; o <<= 1) {
                        if (!PRE) a += __shfl_xor_sync(0xffffffffu, a, o);
                        b += __shfl_xor_sync(0xffffffffu, b, o);
                    }
                }
                const float vj = v_s[tt * DELTA_COLS + col * CPT + j];
                const float u = PRE ? vj : b_s[tt] * (vj - a);
                if (slice == 0 && live[j] && sg.pass != 1)
                    out[((int64_t)(t0 + tt) * H + h) * vdim + column + j] = fmaf(skq[tt], u, b);
#pragma unroll
                for (int i = 0; i < DPT; ++i) S[j][i] = fmaf(e[i].w, u, e[i].z * S[j][i]);
            }
            if (PRE && sg.pass == 1) {
#pragma unroll
                for (int i = 0; i < DPT; ++i) Pd[i] *= e[i].z;
            }
        }
        __syncthreads();                                               // pack and this stage's rows are free again
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    if (sg.pass == 2) return;                                          // the row's end state is delta_fold's
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = slice + DELTA_SLICES * i;
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            if (live[j] && d < dim) S_g[(int64_t)d * vdim + column + j] = S[j][i];
        if (sg.pass == 1 && blockIdx.z == 0 && col == 0 && d < dim)
            sg.seg_decay[(((int64_t)r * sg.nseg + seg) * H + h) * dim + d] = Pd[i];
    }
}

// Per row, head and state entry: the segments' start states from their end states and decays (see above).
__global__ void delta_fold_kernel(float* __restrict__ state, int64_t slot_stride, const int* __restrict__ row_slot,
                                  float* __restrict__ seg_state, const float* __restrict__ seg_decay, int nseg, int H,
                                  int dim, int vdim) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y;
    float* slot = state + (int64_t)row_slot[r] * slot_stride + (int64_t)h * dim * vdim;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < dim * vdim; e += gridDim.z * blockDim.x) {
        const int d = e / vdim;
        float cur = slot[e];
        for (int j = 0; j < nseg; ++j) {
            const int64_t at = ((int64_t)r * nseg + j) * H + h;
            const float end = seg_state[at * dim * vdim + e];
            seg_state[at * dim * vdim + e] = cur;
            cur = fmaf(seg_decay[at * dim + d], cur, end);
        }
        slot[e] = cur;
    }
}

extern "C" int acorn_delta_rule(const float* qn, const float* kn, const float* vv, const float* beta, const float* g,
                                float* state, int64_t slot_stride, const int* row_start, const int* row_slot, float* out,
                                int rows, int H, int KH, int dim, int vdim, const float* bonus, int pass, int nseg,
                                int seg_len, float* seg_state, float* seg_decay, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H > 65535 || vdim > 65535 || dim > 256 || H % KH) return ACORN_ERR_UNSUPPORTED;
    if (bonus == nullptr && beta == nullptr) return ACORN_ERR_UNSUPPORTED;
    DeltaSegments sg = {pass, nseg, seg_len, seg_state, seg_decay};
    if (pass != 0 && (bonus == nullptr || pass < 0 || pass > 2 || nseg < 1 || seg_len < 1 || seg_state == nullptr ||
                      seg_decay == nullptr || (int64_t)rows * nseg > 0x7fffffff))
        return ACORN_ERR_UNSUPPORTED;                   // segments fold only in the form that reads the state first
    const int grid_rows = pass ? rows * nseg : rows;
    const int stage = dim <= 64 ? 32 : (dim <= 128 ? 16 : 8);
#define DELTA_LAUNCH(N, SL)                                                                                                   \
    do {                                                                                                                      \
        if (bonus) DELTA_LAUNCH_AS(N, SL, true, 1, DELTA_THREADS);                                                            \
        DELTA_LAUNCH_AS(N, SL, false, 1, DELTA_THREADS);                                                                      \
    } while (0)
#define DELTA_LAUNCH_AS(N, SL, PRE, CPT, NT)                                                                                  \
    do {                                                                                                                      \
        const int cols = (NT) / (SL) * (CPT);                                                                                 \
        dim3 block(NT);                                                                                                       \
        dim3 grid(grid_rows, H, (vdim + cols - 1) / cols);                                                                    \
        const size_t smem = ((size_t)stage * (N) * (SL) * 4 + (size_t)2 * stage * 3 * dim + 2 * stage * cols + 3 * stage) *    \
                            sizeof(float);                                                                                    \
        static AcornPerDevice configured;                                                                                     \
        if (!configured.seen()) {                                                                                             \
            cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<N, SL, PRE, CPT, NT>,                                      \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,                                 \
                                                 100 * 1024);                                                                 \
            if (e != cudaSuccess) return (int)e;                                                                              \
            configured.mark();                                                                                                \
        }                                                                                                                     \
        return acorn_launch(delta_rule_kernel<N, SL, PRE, CPT, NT>, grid, block, smem, stream, qn, kn, vv, beta, g, state,    \
                            slot_stride, row_start, row_slot, out, H, KH, dim, vdim, stage, bonus, sg);                       \
    } while (0)
    // a thread holds few state entries (4; 8 for the widest heads): a warp is alone on its scheduler, so the
    // time of a token is the number of instructions a thread issues for it, and spreading a column over more
    // lanes (up to a whole warp) shortens it although the reduction grows
    // (the tokens' staging is shared by a block's columns: 256 threads keep 8 to 64 columns together)
    // rows in segments: the device is full of blocks, so what counts is the work all of them do for a token, and of
    // that the reads of the packed entries from shared memory weigh most: a column over fewer lanes (more entries a
    // thread, more columns a warp, which share the entries they read) and several columns a thread cut them down
    if (pass != 0) {
        if (dim <= 32) DELTA_LAUNCH_AS(8, 4, true, 1, 256);
        if (dim <= 64) DELTA_LAUNCH_AS(8, 8, true, 4, 128);
        if (dim <= 128) DELTA_LAUNCH_AS(16, 8, true, 2, 256);
        DELTA_LAUNCH_AS(16, 16, true, 1, 256);
    }
    if (dim <= 16) DELTA_LAUNCH(4, 4);
    if (dim <= 32) DELTA_LAUNCH(4, 8);
    if (dim <= 64) DELTA_LAUNCH(4, 16);
    if (dim <= 128) DELTA_LAUNCH(8, 16);
    DELTA_LAUNCH(8, 32);
#undef DELTA_LAUNCH
#undef DELTA_LAUNCH_AS
}

extern "C" int acorn_delta_fold(float* state, int64_t slot_stride, const int* row_slot, float* seg_state,
                                const float* seg_decay, int rows, int nseg, int H, int dim, int vdim, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H > 65535 || nseg < 1) return ACORN_ERR_UNSUPPORTED;
    int bz = (dim * vdim + 255) / 256;
    if (bz > 64) bz = 64;
    return acorn_launch(delta_fold_kernel, dim3(rows, H, bz), dim3(256), 0, stream, state, slot_stride, row_slot, seg_state,
                        seg_decay, nseg, H, dim, vdim);
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * gate   (w [vdim] shared by the heads: w_heads = 1; or one
// per head, [H, vdim]: w_heads = H)
template <typename T>
__global__ void delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, const float* __restrict__ w_,
                                 T* __restrict__ y, int vdim, float eps, int64_t total_heads, int w_heads) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t th = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // token * H + head
    if (th >= total_heads) return;
    const float* row = o + th * vdim;
    const float* w = w_ + (th % w_heads) * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += row[j] * row[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) y[th * vdim + j] = from_float<T>(row[j] * inv * w[j] * gate[th * vdim + j]);
}

extern "C" int acorn_delta_out(const float* o, const float* gate, const float* w, void* y, int tokens, int H, int vdim,
                               float eps, int dtype, int w_per_head, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * H;
    if (total <= 0) return 0;
    const int64_t blocks = (total + 3) / 4;
    if (blocks > 0x7fffffff) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(delta_out_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, o,
                                                       gate, w, (T*)y, vdim, eps, total, w_per_head ? H : 1));
    return ACORN_ERR_UNSUPPORTED;
}
