// Time mixing with a matrix state per head (the RWKV kind): the pieces around the recurrence, which is
// the PRE form of delta_rule (delta_rule.cu), and whose output step is delta_out with a weight per head.
//
//   token_shift   per token: n blends of the token's row h and the row before it in its request,
//                     out[s][t] = h[t] + (prev[t] - h[t]) * mu[s],
//                 prev of a step's first token from the request's state slot (float32 [W] at an offset:
//                 the last row of the step before, zeros when the request starts; conv_state_update with
//                 two taps keeps it; with update_single the kernel itself puts the row of a request that brings
//                 a single token into its slot, and that kernel then skips such rows).  One rounding to the
//                 activation type.
//   wkv_prep      per token: float32 copies of r, k, v for the recurrence, the decay
//                 exp(-exp(z + w0)) per head and key channel and the gate silu(g), all float32.
#include "common.cuh"

#define SHIFT_MAX_BLENDS 8

template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, int64_t ld, const float* __restrict__ mu,
                                   float* __restrict__ state, int64_t slot_stride, int64_t prev_off,
                                   const int* __restrict__ token_row, const int* __restrict__ row_start,
                                   const int* __restrict__ row_slot, T* __restrict__ out, int64_t tokens, int W, int n,
                                   int update_single) {
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    const int r = token_row[t];
    const bool first = t == row_start[r];
    const bool keep = update_single && first && row_start[r + 1] == t + 1;      // the row's only token: it is the next step's prev
    float* ps = state + (int64_t)row_slot[r] * slot_stride + prev_off;
    const T* cur = h + t * ld;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float x = to_float(cur[i]);
        const float p = first ? ps[i] : to_float(cur[i - ld]);
        const float d = p - x;
        if (keep) ps[i] = x;
#pragma unroll
        for (int s = 0; s < SHIFT_MAX_BLENDS; ++s)
            if (s < n) out[((int64_t)s * tokens + t) * W + i] = from_float<T>(fmaf(d, mu[(int64_t)s * W + i], x));
    }
}

// The same, four channels a thread (8- or 16-byte accesses): widths, row strides and state offsets that are
// multiples of four.
template <typename T>
__global__ void token_shift_vec_kernel(const T* __restrict__ h, int64_t ld, const float* __restrict__ mu,
                                       float* __restrict__ state, int64_t slot_stride, int64_t prev_off,
                                       const int* __restrict__ token_row, const int* __restrict__ row_start,
                                       const int* __restrict__ row_slot, T* __restrict__ out, int64_t tokens, int W,
                                       int n, int update_single) {
    pdl_wait();
    pdl_trigger();
    const int i = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (i >= W) return;
    const int64_t t = blockIdx.x;
    const int r = token_row[t];
    const bool first = t == row_start[r];
    const bool keep = update_single && first && row_start[r + 1] == t + 1;
    float* ps = state + (int64_t)row_slot[r] * slot_stride + prev_off + i;
    const T* cur = h + t * ld + i;
    const float4 x = Vec4<T>::load(cur);
    const float4 p = first ? *reinterpret_cast<const float4*>(ps) : Vec4<T>::load(cur - ld);
    const float4 d = make_float4(p.x - x.x, p.y - x.y, p.z - x.z, p.w - x.w);
    if (keep) *reinterpret_cast<float4*>(ps) = x;
#pragma unroll
    for (int s = 0; s < SHIFT_MAX_BLENDS; ++s)
        if (s < n) {
            const float4 m = *reinterpret_cast<const float4*>(mu + (int64_t)s * W + i);
            Vec4<T>::store(out + ((int64_t)s * tokens + t) * W + i,
                           make_float4(fmaf(d.x, m.x, x.x), fmaf(d.y, m.y, x.y), fmaf(d.z, m.z, x.z), fmaf(d.w, m.w, x.w)));
        }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int acorn_token_shift(const void* h, int64_t ld, const float* mu, float* state, int64_t slot_stride,
                                 int64_t prev_off, const int* token_row, const int* row_start, const int* row_slot,
                                 void* out, int tokens, int W, int n, int dtype, int update_single, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (n < 1 || n > SHIFT_MAX_BLENDS) return ACORN_ERR_UNSUPPORTED;
    if (W % 4 == 0 && ld % 4 == 0 && slot_stride % 4 == 0 && prev_off % 4 == 0 && (W + 511) / 512 <= 65535 &&
        aligned16(h) && aligned16(mu) && aligned16(state) && aligned16(out)) {
        const int lanes = (W / 4 + 31) / 32 * 32;
        const int threads_v = lanes < 128 ? lanes : 128;
        dim3 grid(tokens, (W / 4 + threads_v - 1) / threads_v);
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(token_shift_vec_kernel<T>, grid, dim3(threads_v), 0, stream,
                                                           (const T*)h, ld, mu, state, slot_stride, prev_off, token_row,
                                                           row_start, row_slot, (T*)out, (int64_t)tokens, W, n,
                                                           update_single));
    }
    const int threads = W >= 1024 ? 256 : 128;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(token_shift_kernel<T>, dim3(tokens), dim3(threads), 0, stream,
                                                       (const T*)h, ld, mu, state, slot_stride, prev_off, token_row,
                                                       row_start, row_slot, (T*)out, (int64_t)tokens, W, n, update_single));
    return ACORN_ERR_UNSUPPORTED;
}

// r, k, v, g: [T, C] of the activation type (row strides in elements); z: [T, C] float32, the decay's
// pre-activation without its constant part w0 [C].
template <typename T>
__global__ void wkv_prep_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                const T* __restrict__ g, int64_t ld, const float* __restrict__ z, int64_t ld_z,
                                const float* __restrict__ w0, float* __restrict__ r32, float* __restrict__ k32,
                                float* __restrict__ v32, float* __restrict__ decay, float* __restrict__ gate, int C) {
    pdl_wait();
    pdl_trigger();
    const int64_t t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int64_t in = t * ld + c, o = t * C + c;
    r32[o] = to_float(r[in]);
    k32[o] = to_float(k[in]);
    v32[o] = to_float(v[in]);
    const float gv = to_float(g[in]);
    gate[o] = gv / (1.f + expf(-gv));
    decay[o] = expf(-expf(z[t * ld_z + c] + w0[c]));
}

extern "C" int acorn_wkv_prep(const void* r, const void* k, const void* v, const void* g, int64_t ld, const float* z,
                              int64_t ld_z, const float* w0, float* r32, float* k32, float* v32, float* decay,
                              float* gate, int tokens, int C, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if ((C + 127) / 128 > 65535) return ACORN_ERR_UNSUPPORTED;
    dim3 grid(tokens, (C + 127) / 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(wkv_prep_kernel<T>, grid, dim3(128), 0, stream, (const T*)r,
                                                       (const T*)k, (const T*)v, (const T*)g, ld, z, ld_z, w0, r32, k32,
                                                       v32, decay, gate, C));
    return ACORN_ERR_UNSUPPORTED;
}
