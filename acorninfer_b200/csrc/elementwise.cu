// Embedding lookup, fused residual-add + RMSNorm, SwiGLU.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out32[t, :] = table[ids[t], :] * scale   (float32 residual stream)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out32, int H, float scale) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const T* row = table + (int64_t)ids[t] * H;
    float* o = out32 + (int64_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

extern "C" int acorn_embed(const int* ids, const void* table, float* out32, int tokens, int H,
                           int dtype, float scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(embed_kernel<T>, dim3(tokens), dim3(256), 0, stream, ids, (const T*)table, out32, H, scale));
    return ACORN_ERR_UNSUPPORTED;
}

// token_ids[dst[i]] = src_tokens[src[i]]: the ids a step decodes from are the ids the step before it
// sampled, taken on the device (the host reads them one step later).
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ dst,
                                    const int* __restrict__ src, const int* __restrict__ src_tokens, int n) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) token_ids[dst[i]] = src_tokens[src[i]];
}

extern "C" int acorn_patch_tokens(int* token_ids, const int* dst, const int* src, const int* src_tokens, int n,
                                  cudaStream_t stream) {
    if (n <= 0) return 0;
    return acorn_launch(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, token_ids, dst, src,
                        src_tokens, n);
}

// ---------------------------------------------------------------- add + RMSNorm
// v = resid32[row] (+ delta[row]);  if write_resid: resid32[row] = v
// out[r] = v * rsqrt(mean(v^2) + eps) * w          (all in float32, one rounding)
// row = row_idx ? row_idx[r] : r.  With row_idx the residual is not written back
// (a row may be listed twice).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid32, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int* __restrict__ row_idx, int H, float eps) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const int64_t row = row_idx ? row_idx[r] : r;
    const bool write_resid = (row_idx == nullptr) && (delta != nullptr);
    float* x = resid32 + row * H;
    const T* dl = delta ? delta + row * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl) v += to_float(dl[i]);
        if (write_resid) x[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    T* o = out + (int64_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl && !write_resid) v += to_float(dl[i]);
        o[i] = from_float<T>(v * inv * w[i]);
    }
}

// The same with four elements per thread and step, the row kept in registers between the two
// passes: for widths that are a multiple of 4 and at most threads * 4 * RMS_MAX_ITER.
#define RMS_MAX_ITER 8

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid32, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ out,
                                       const int* __restrict__ row_idx, int H, float eps) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const int64_t row = row_idx ? row_idx[r] : r;
    const bool write_resid = (row_idx == nullptr) && (delta != nullptr);
    float* x = resid32 + row * H;
    const T* dl = delta ? delta + row * H : nullptr;
    float4 v[RMS_MAX_ITER];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < RMS_MAX_ITER; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            float4 a = *reinterpret_cast<const float4*>(x + i);
            if (dl) {
                const float4 d = Vec4<T>::load(dl + i);
                a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
            }
            if (write_resid) *reinterpret_cast<float4*>(x + i) = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            v[it] = a;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    T* o = out + (int64_t)r * H;
#pragma unroll
    for (int it = 0; it < RMS_MAX_ITER; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < H) {
            const float4 ww = *reinterpret_cast<const float4*>(w + i);
            Vec4<T>::store(o + i, make_float4(v[it].x * inv * ww.x, v[it].y * inv * ww.y, v[it].z * inv * ww.z,
                                              v[it].w * inv * ww.w));
        }
    }
}

extern "C" int acorn_add_rmsnorm(float* resid32, const void* delta, const float* w, void* out,
                                 const int* row_idx, int rows, int H, float eps, int dtype,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H % 4 == 0) {
        int threads = ((H / 4 + 31) / 32) * 32;
        if (threads > 256) threads = 256;
        if ((int64_t)threads * 4 * RMS_MAX_ITER >= H) {
            ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_rmsnorm_vec_kernel<T>, dim3(rows), dim3(threads), 0,
                                                               stream, resid32, (const T*)delta, w, (T*)out, row_idx,
                                                               H, eps));
        }
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_rmsnorm_kernel<T>, dim3(rows), dim3(threads), 0, stream,
                                                       resid32, (const T*)delta, w, (T*)out, row_idx, H, eps));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- gated linear unit (SwiGLU, GeGLU)
// out[t, i] = act(gate) * up;  act 0: silu(z) = z / (1 + exp(-z)),  act 1: the tanh form of gelu,
// 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) = z sigmoid(2 sqrt(2/pi) (z + 0.044715 z^3)).  A row of gu holds, per block of b
// outputs, b gate values then b up values: gate of output i at (i / b) * 2b + i % b, up b further.
// b = I is the plain layout [gate | up].
// act 2, the capped form with `limit` L: g = min(gate, L), u = clamp(up, -L, L), out = g sigmoid(1.702 g) (u + 1).
__device__ __forceinline__ float glu_act(float g, int act) {
    if (act == 2) return g / (1.f + expf(-1.702f * g));          // the capped form's gate (the caps are the caller's)
    if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}

// the same by the fast float32 instructions (relative error about 2^-22), for results rounded to bfloat16
template <int ACT> __device__ __forceinline__ float glu_act_fast(float g) {
    const float z = ACT == 1 ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : (ACT == 2 ? 1.702f * g : g);
    return __fdividef(g, 1.f + __expf(-z));
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int I, int b, int act,
                              float limit) {
    pdl_wait();
    pdl_trigger();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        const int64_t gi = t * 2 * I + (int64_t)(i / b) * 2 * b + i % b;
        float g = to_float(gu[gi]);
        float u = to_float(gu[gi + b]);
        if (act == 2) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit) + 1.f;
        }
        out[idx] = from_float<T>(glu_act(g, act) * u);
    }
}

// bfloat16 rows whose block width b is a multiple of 8: 16-byte loads and stores (b8 = b / 8).
// blockIdx.y is the token, so that no index is divided by the row width; a thread takes two
// 16-byte chunks of outputs a step (four loads in flight).
template <int ACT>
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I8, int b8, float limit) {
    pdl_wait();
    pdl_trigger();
    const bf16* row = gu + (int64_t)blockIdx.y * I8 * 16;
    bf16* orow = out + (int64_t)blockIdx.y * I8 * 8;
    auto one = [&](const uint4& g4, const uint4& u4) -> uint4 {
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
            float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[k]));
            if (ACT == 2) {         // the capped form
                g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
                u.x = fminf(fmaxf(u.x, -limit), limit) + 1.f; u.y = fminf(fmaxf(u.y, -limit), limit) + 1.f;
            }
            // exp and the quotient by the fast float32 instructions (relative error about 2^-22, far below
            // the bfloat16 rounding of the result): with the exact ones the kernel is bound by arithmetic
            __nv_bfloat162 o = __floats2bfloat162_rn(glu_act_fast<ACT>(g.x) * u.x, glu_act_fast<ACT>(g.y) * u.y);
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        return make_uint4(ow[0], ow[1], ow[2], ow[3]);
    };
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I8; i += 2 * stride) {
        const int i2 = i + stride;
        const int gi = (i / b8) * 2 * b8 + i % b8;
        const uint4 g4 = *reinterpret_cast<const uint4*>(row + (int64_t)gi * 8);
        const uint4 u4 = *reinterpret_cast<const uint4*>(row + (int64_t)(gi + b8) * 8);
        if (i2 < I8) {
            const int gj = (i2 / b8) * 2 * b8 + i2 % b8;
            const uint4 g5 = *reinterpret_cast<const uint4*>(row + (int64_t)gj * 8);
            const uint4 u5 = *reinterpret_cast<const uint4*>(row + (int64_t)(gj + b8) * 8);
            *reinterpret_cast<uint4*>(orow + (int64_t)i2 * 8) = one(g5, u5);
        }
        *reinterpret_cast<uint4*>(orow + (int64_t)i * 8) = one(g4, u4);
    }
}

extern "C" int acorn_swiglu(const void* gu, void* out, int tokens, int I, int block, int dtype, int act, float limit,
                            cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * I;
    if (total <= 0) return 0;
    if (block <= 0 || I % block != 0 || act < 0 || act > 2) return ACORN_ERR_UNSUPPORTED;
    if (dtype == ACORN_DTYPE_BF16 && block % 8 == 0 && tokens <= 65535) {
        const int I8 = I / 8;
        int bx = (I8 + 511) / 512;                  // 256 threads, two chunks each
        if (bx < 1) bx = 1;
        if (act == 2)
            return acorn_launch(swiglu_bf16x8_kernel<2>, dim3(bx, tokens), dim3(256), 0, stream, (const bf16*)gu,
                                (bf16*)out, I8, block / 8, limit);
        if (act == 1)
            return acorn_launch(swiglu_bf16x8_kernel<1>, dim3(bx, tokens), dim3(256), 0, stream, (const bf16*)gu,
                                (bf16*)out, I8, block / 8, limit);
        return acorn_launch(swiglu_bf16x8_kernel<0>, dim3(bx, tokens), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out,
                            I8, block / 8, limit);
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                       (const T*)gu, (T*)out, total, I, block, act, limit));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- plain activations
// out = act(x) elementwise: 0 the square of relu, 1 tanh, 2 the tanh form of gelu, 3 silu.  float32 arithmetic,
// one rounding.  x [rows, n] with a row stride; out contiguous.
__device__ __forceinline__ float plain_act(float z, int act) {
    switch (act) {
        case 0: { const float r = fmaxf(z, 0.f); return r * r; }
        case 1: return tanhf(z);
        case 2: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        default: return z / (1.f + expf(-z));
    }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, int64_t ld, T* __restrict__ out, int n, int act) {
    pdl_wait();
    pdl_trigger();
    const int64_t row = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x)
        out[row * n + i] = from_float<T>(plain_act(to_float(x[row * ld + i]), act));
}

// bfloat16 rows of a width that is a multiple of 8 and 16-byte aligned: eight elements a thread and step
__global__ void activation_bf16x8_kernel(const bf16* __restrict__ x, int64_t ld, bf16* __restrict__ out, int n8, int act) {
    pdl_wait();
    pdl_trigger();
    const int64_t row = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n8; i += gridDim.y * blockDim.x) {
        const uint4 in = *reinterpret_cast<const uint4*>(x + row * ld + (int64_t)i * 8);
        const uint32_t iw[4] = {in.x, in.y, in.z, in.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&iw[k]));
            __nv_bfloat162 o = __floats2bfloat162_rn(plain_act(f.x, act), plain_act(f.y, act));
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        *reinterpret_cast<uint4*>(out + (row * n8 + i) * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

extern "C" int acorn_activation(const void* x, int64_t ld, void* out, int rows, int n, int act, int dtype,
                                cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (act < 0 || act > 3) return ACORN_ERR_UNSUPPORTED;
    if (dtype == ACORN_DTYPE_BF16 && n % 8 == 0 && ld % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        int by = (n / 8 + 255) / 256;
        if (by > 64) by = 64;
        return acorn_launch(activation_bf16x8_kernel, dim3(rows, by), dim3(256), 0, stream, (const bf16*)x, ld, (bf16*)out,
                            n / 8, act);
    }
    int by = (n + 255) / 256;
    if (by > 64) by = 64;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(activation_kernel<T>, dim3(rows, by), dim3(256), 0, stream,
                                                       (const T*)x, ld, (T*)out, n, act));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- a token's own side rows, gated
// out[t, i] = gelu_tanh(z[t, i]) * table[ids[t], col0 + i]: columns col0 .. col0 + n of the token's row of a
// side table, gated by a projection z of the stream.  float32 arithmetic, one rounding.
template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ z, const int* __restrict__ ids, const T* __restrict__ table,
                                 int64_t ld_table, int col0, T* __restrict__ out, int64_t total, int n) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t t = idx / n;
    const int i = (int)(idx - t * n);
    const float e = to_float(table[(int64_t)ids[t] * ld_table + col0 + i]);
    out[idx] = from_float<T>(plain_act(to_float(z[idx]), 2) * e);
}

extern "C" int acorn_side_gate(const void* z, const int* ids, const void* table, int64_t ld_table, int col0, void* out,
                               int tokens, int n, int dtype, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * n;
    if (total <= 0) return 0;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffff) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(side_gate_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream,
                                                       (const T*)z, ids, (const T*)table, ld_table, col0, (T*)out, total, n));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- casts
template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_float<B>(to_float(in[i]));
}

// dtype_in -> dtype_out over n contiguous elements.
extern "C" int acorn_cast(const void* in, void* out, int64_t n, int dtype_in, int dtype_out, cudaStream_t stream) {
    if (n <= 0) return 0;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype_in == ACORN_DTYPE_BF16 && dtype_out == ACORN_DTYPE_F32)
        cast_kernel<bf16, float><<<(int)blocks, 256, 0, stream>>>((const bf16*)in, (float*)out, n);
    else if (dtype_in == ACORN_DTYPE_F32 && dtype_out == ACORN_DTYPE_BF16)
        cast_kernel<float, bf16><<<(int)blocks, 256, 0, stream>>>((const float*)in, (bf16*)out, n);
    else
        return ACORN_ERR_UNSUPPORTED;
    return acorn_launch_status();
}

// ---------------------------------------------------------------- hashed bigram rows
// resid32[t] += table[row(t)]: row = (prev * mul_prev + cur * mul_cur) mod buckets, where prev is the token
// before t in its request; a request's first token takes row `buckets`.  The token before a row's
// first token is the request's state (prev_state[slot], the last token of its previous step); the block
// of a row's first token reads it and then stores the row's last token there.
template <typename T>
__global__ void bigram_add_kernel(float* __restrict__ resid32, const int* __restrict__ token_ids,
                                  const int* __restrict__ token_row, const int* __restrict__ row_start,
                                  const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                                  int* __restrict__ prev_state, const T* __restrict__ table, int H, int buckets,
                                  int mul_prev, int mul_cur) {
    __shared__ int s_row;
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        const int r = token_row[t], first = row_start[r];
        const int cur = token_ids[t];
        int row;
        if (t > first) {
            row = (int)(((int64_t)token_ids[t - 1] * mul_prev + (int64_t)cur * mul_cur) % buckets);
        } else {
            const int slot = row_slot[r];
            row = row_pos[r] == 0 ? buckets
                                  : (int)(((int64_t)prev_state[slot] * mul_prev + (int64_t)cur * mul_cur) % buckets);
            prev_state[slot] = token_ids[row_start[r + 1] - 1];
        }
        s_row = row;
    }
    __syncthreads();
    const T* src = table + (int64_t)s_row * H;
    float* o = resid32 + (int64_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] += to_float(src[i]);
}

extern "C" int acorn_bigram_add(float* resid32, const int* token_ids, const int* token_row, const int* row_start,
                                const int* row_pos, const int* row_slot, int* prev_state, const void* table,
                                int tokens, int H, int buckets, int mul_prev, int mul_cur, int dtype,
                                cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (buckets < 1) return ACORN_ERR_UNSUPPORTED;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(bigram_add_kernel<T>, dim3(tokens), dim3(128), 0, stream, resid32,
                                                       token_ids, token_row, row_start, row_pos, row_slot, prev_state,
                                                       (const T*)table, H, buckets, mul_prev, mul_cur));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- RMSNorm of a sublayer's output, added
// resid32[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w   (float32), and, if `rounded` is given, the new
// residual row rounded to T: what the next sublayer reads.
template <typename T>
__global__ void rmsnorm_add_kernel(float* __restrict__ resid32, const T* __restrict__ y, const float* __restrict__ w,
                                   T* __restrict__ rounded, int H, float eps) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int64_t row = blockIdx.x;
    const T* yr = y + row * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_float(yr[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    float* x = resid32 + row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = x[i] + to_float(yr[i]) * inv * w[i];
        x[i] = v;
        if (rounded) rounded[row * H + i] = from_float<T>(v);
    }
}

// Both of the above, four entries a thread and access (8 or 16 bytes), a thread's part of the row in registers
// (NV vectors) from the first read to the last write: widths that are multiples of four, up to 16 NV threads.
// NEXT: the second norm follows (`out` is then the normed row, else the rounded new residual or null).
template <typename T, int NV, bool NEXT>
__global__ void rmsnorm_add_vec_kernel(float* __restrict__ resid32, const T* __restrict__ y, const float* __restrict__ w,
                                       const float* __restrict__ w_next, T* __restrict__ out, int H, float eps,
                                       float eps_next) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int64_t row = blockIdx.x;
    const int n4 = H >> 2;
    const T* yr = y + row * H;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < n4 ? Vec4<T>::load(yr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    float* x = resid32 + row * H;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 r = *reinterpret_cast<const float4*>(x + 4 * i);
            const float4 g = *reinterpret_cast<const float4*>(w + 4 * i);
            v[k] = make_float4(r.x + v[k].x * inv * g.x, r.y + v[k].y * inv * g.y, r.z + v[k].z * inv * g.z,
                               r.w + v[k].w * inv * g.w);
            *reinterpret_cast<float4*>(x + 4 * i) = v[k];
            if (!NEXT && out) Vec4<T>::store(out + row * H + 4 * i, v[k]);
            s2 += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    if (!NEXT) return;
    s2 = block_sum(s2, scratch);
    const float inv2 = rsqrtf(s2 / (float)H + eps_next);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 g = *reinterpret_cast<const float4*>(w_next + 4 * i);
            Vec4<T>::store(out + row * H + 4 * i,
                           make_float4(v[k].x * inv2 * g.x, v[k].y * inv2 * g.y, v[k].z * inv2 * g.z, v[k].w * inv2 * g.w));
        }
    }
}

// 0: launched; -1: not a case of the vector form
template <bool NEXT>
static int launch_rmsnorm_add_vec(float* resid32, const void* y, const float* w, const float* w_next, void* out, int rows,
                                  int H, float eps, float eps_next, int dtype, cudaStream_t stream, int* status) {
    const uintptr_t all = (uintptr_t)resid32 | (uintptr_t)y | (uintptr_t)w | (uintptr_t)w_next | (uintptr_t)out;
    if (H % 4 != 0 || (all & 15) != 0) return -1;
    const int n4 = H / 4;
    const int threads = n4 <= 256 ? (n4 + 31) / 32 * 32 : (n4 <= 1024 ? 256 : 512);
    const int nv = (n4 + threads - 1) / threads;
    if (nv > 4) return -1;
#define NORM_VEC(NV)                                                                                                   \
    ACORN_DISPATCH_DTYPE(dtype, T, *status = acorn_launch(rmsnorm_add_vec_kernel<T, NV, NEXT>, dim3(rows), dim3(threads), \
                                                          0, stream, resid32, (const T*)y, w, w_next, (T*)out, H, eps,  \
                                                          eps_next))
    if (nv == 1) NORM_VEC(1);
    else if (nv == 2) NORM_VEC(2);
    else NORM_VEC(4);
#undef NORM_VEC
    return 0;
}

extern "C" int acorn_rmsnorm_add(float* resid32, const void* y, const float* w, void* rounded, int rows, int H,
                                 float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    int status = 0;
    if (launch_rmsnorm_add_vec<false>(resid32, y, w, nullptr, rounded, rows, H, eps, 0.f, dtype, stream, &status) == 0)
        return status;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(rmsnorm_add_kernel<T>, dim3(rows), dim3(threads), 0, stream, resid32,
                                                       (const T*)y, w, (T*)rounded, H, eps));
    return ACORN_ERR_UNSUPPORTED;
}

// The same, followed at once by the norm the next sublayer reads the stream through:
//   x = resid32[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w;   normed[t] = x * rsqrt(mean(x^2) + eps_next) * w_next
// (a sublayer's output norm and the next sublayer's input norm in one pass over the row; the updated row
// waits in shared memory between the two reductions).
template <typename T>
__global__ void rmsnorm_add_norm_kernel(float* __restrict__ resid32, const T* __restrict__ y, const float* __restrict__ w,
                                        const float* __restrict__ w_next, T* __restrict__ normed, int H, float eps,
                                        float eps_next) {
    extern __shared__ float xrow[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int64_t row = blockIdx.x;
    const T* yr = y + row * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_float(yr[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    float* x = resid32 + row * H;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = x[i] + to_float(yr[i]) * inv * w[i];
        x[i] = v;
        xrow[i] = v;
        s2 += v * v;
    }
    __syncthreads();                                    // scratch is read by all before it is written again
    s2 = block_sum(s2, scratch);
    const float inv2 = rsqrtf(s2 / (float)H + eps_next);
    for (int i = threadIdx.x; i < H; i += blockDim.x) normed[row * H + i] = from_float<T>(xrow[i] * inv2 * w_next[i]);
}

extern "C" int acorn_rmsnorm_add_norm(float* resid32, const void* y, const float* w, const float* w_next, void* normed,
                                      int rows, int H, float eps, float eps_next, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    int status = 0;
    if (launch_rmsnorm_add_vec<true>(resid32, y, w, w_next, normed, rows, H, eps, eps_next, dtype, stream, &status) == 0)
        return status;
    if ((size_t)H * sizeof(float) > 48 * 1024) return ACORN_ERR_UNSUPPORTED;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(rmsnorm_add_norm_kernel<T>, dim3(rows), dim3(threads),
                                                       (size_t)H * sizeof(float), stream, resid32, (const T*)y, w, w_next,
                                                       (T*)normed, H, eps, eps_next));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- add + LayerNorm (weight and bias)
// v = resid32[row] (+ delta[row]) (+ delta2[row]);  if write_resid: resid32[row] = v
// out[r] = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * w + b      (float32, one rounding)
// row = row_idx ? row_idx[r] : r; with row_idx the residual is not written back.  Two deltas: the two
// sublayers of a block whose mixer and feed-forward read the same normed rows.  The row is kept in
// shared memory between the passes; the variance is taken of the deviations (two passes), not as
// mean(v^2) - mean(v)^2.
template <typename T>
__global__ void add_layernorm_kernel(float* __restrict__ resid32, const T* __restrict__ delta,
                                     const T* __restrict__ delta2, const float* __restrict__ w,
                                     const float* __restrict__ b, T* __restrict__ out,
                                     const int* __restrict__ row_idx, int H, float eps) {
    extern __shared__ float rowv[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const int64_t row = row_idx ? row_idx[r] : r;
    const bool write_resid = (row_idx == nullptr) && (delta != nullptr || delta2 != nullptr);
    float* x = resid32 + row * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (delta) v += to_float(delta[row * H + i]);
        if (delta2) v += to_float(delta2[row * H + i]);
        if (write_resid) x[i] = v;
        rowv[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float dv = rowv[i] - mean;
        ss += dv * dv;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    T* o = out + (int64_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_float<T>((rowv[i] - mean) * inv * w[i] + (b ? b[i] : 0.f));
}

extern "C" int acorn_add_layernorm(float* resid32, const void* delta, const void* delta2, const float* w,
                                   const float* b, void* out, const int* row_idx, int rows, int H, float eps,
                                   int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if ((size_t)H * sizeof(float) > 48 * 1024) return ACORN_ERR_UNSUPPORTED;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_layernorm_kernel<T>, dim3(rows), dim3(threads),
                                                       (size_t)H * sizeof(float), stream, resid32, (const T*)delta,
                                                       (const T*)delta2, w, b, (T*)out, row_idx, H, eps));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- resid32 += delta
template <typename T>
__global__ void add_into_kernel(float* __restrict__ resid32, const T* __restrict__ delta, int64_t n) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        resid32[i] += to_float(delta[i]);
}

extern "C" int acorn_add_into(float* resid32, const void* delta, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(add_into_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                       resid32, (const T*)delta, n));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- a gate per head
// out[t, h, :] = x[t, h, :] * scale * sigmoid(g[t * ldg + h]): every head's output times one number of its
// own, a function of the layer's input (g is a slice of a wider product; null: times scale); float32, one
// rounding.  out may be x itself, or rows of another buffer (row stride ldo).
template <typename T>
__global__ void head_gate_kernel(const T* x, const T* __restrict__ g, int64_t ldg, T* out, int64_t ldo, int heads,
                                 int d, int64_t total, float scale) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t th = i / d;
        const int64_t t = th / heads;
        const int h = (int)(th - t * heads);
        const float f = g ? scale / (1.f + expf(-to_float(g[t * ldg + h]))) : scale;
        out[t * ldo + (i - t * heads * d)] = from_float<T>(to_float(x[i]) * f);
    }
}

// The same, 16 bytes of a head to a thread (head sizes and row strides that are multiples of 16 bytes).
template <typename T>
__global__ void head_gate_vec_kernel(const T* x, const T* __restrict__ g, int64_t ldg, T* out, int64_t ldo, int heads,
                                     int d, int64_t total_vecs, float scale) {
    constexpr int VEC = 16 / (int)sizeof(T);
    pdl_wait();
    pdl_trigger();
    const int row_vecs = heads * d / VEC, head_vecs = d / VEC;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / row_vecs;
        const int in_row = (int)(i - t * row_vecs);
        const float f = g ? scale / (1.f + expf(-to_float(g[t * ldg + in_row / head_vecs]))) : scale;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + t * (int64_t)heads * d + (int64_t)in_row * VEC);
        const T* v = reinterpret_cast<const T*>(&raw);
        uint4 res;
        T* o = reinterpret_cast<T*>(&res);
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = from_float<T>(to_float(v[k]) * f);
        *reinterpret_cast<uint4*>(out + t * ldo + (int64_t)in_row * VEC) = res;
    }
}

extern "C" int acorn_head_gate(const void* x, const void* g, int64_t ldg, void* out, int64_t ldo, int tokens, int heads,
                               int d, float scale, int dtype, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * heads * d;
    if (total <= 0) return 0;
    const int vec = dtype == ACORN_DTYPE_F32 ? 4 : 8;
    if (d % vec == 0 && ldo % vec == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int64_t vecs = total / vec;
        int64_t blocks = (vecs + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(head_gate_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                           (const T*)x, (const T*)g, ldg, (T*)out, ldo, heads, d, vecs,
                                                           scale));
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(head_gate_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                                       (const T*)x, (const T*)g, ldg, (T*)out, ldo, heads, d, total,
                                                       scale));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- two score maps of a head into one output
// a [tokens, heads, 2, dv]: the outputs a1, a2 of a head's two attention maps over the same values.
//   o = a1 - lambda a2;   o <- o / sqrt(mean(o^2) + eps) * scale;   out[t, h, :] = o * sigmoid(g[t * ldg + h dv + :])
// (g: a slice of a wider product, a gate per output entry; null: no gate).  float32, one rounding.  A warp a
// (token, head).
template <typename T>
__global__ void diff_combine_kernel(const T* __restrict__ a, const T* __restrict__ g, int64_t ldg, T* __restrict__ out,
                                    int64_t items, int heads, int dv, float lambda, float scale, float eps) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int64_t t = item / heads;
    const int h = (int)(item - t * heads);
    const T* a1 = a + item * 2 * dv;
    const T* a2 = a1 + dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
        const float o = to_float(a1[i]) - lambda * to_float(a2[i]);
        ss += o * o;
    }
    ss = warp_sum(ss);
    const float f = rsqrtf(ss / (float)dv + eps) * scale;
    for (int i = lane; i < dv; i += 32) {
        float o = (to_float(a1[i]) - lambda * to_float(a2[i])) * f;
        if (g) o = o / (1.f + expf(-to_float(g[t * ldg + (int64_t)h * dv + i])));
        out[item * dv + i] = from_float<T>(o);
    }
}

// The same for value rows that are multiples of four up to 512 with aligned rows: four entries a lane (8- or 16-byte
// accesses), the lane's part of the row in registers between the sum of squares and the write.
template <typename T>
__global__ void diff_combine_vec_kernel(const T* __restrict__ a, const T* __restrict__ g, int64_t ldg, T* __restrict__ out,
                                        int64_t items, int heads, int dv, float lambda, float scale, float eps) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int64_t t = item / heads;
    const int h = (int)(item - t * heads);
    const T* a1 = a + item * 2 * dv;
    const T* a2 = a1 + dv;
    float4 o[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = (u * 32 + lane) * 4;
        o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < dv) {
            const float4 x = Vec4<T>::load(a1 + i), y = Vec4<T>::load(a2 + i);
            o[u] = make_float4(x.x - lambda * y.x, x.y - lambda * y.y, x.z - lambda * y.z, x.w - lambda * y.w);
            ss += o[u].x * o[u].x + o[u].y * o[u].y + o[u].z * o[u].z + o[u].w * o[u].w;
        }
    }
    ss = warp_sum(ss);
    const float f = rsqrtf(ss / (float)dv + eps) * scale;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = (u * 32 + lane) * 4;
        if (i < dv) {
            float4 r = make_float4(o[u].x * f, o[u].y * f, o[u].z * f, o[u].w * f);
            if (g) {
                const float4 z = Vec4<T>::load(g + t * ldg + (int64_t)h * dv + i);
                r.x /= 1.f + expf(-z.x); r.y /= 1.f + expf(-z.y); r.z /= 1.f + expf(-z.z); r.w /= 1.f + expf(-z.w);
            }
            Vec4<T>::store(out + item * dv + i, r);
        }
    }
}

extern "C" int acorn_diff_combine(const void* a, const void* g, int64_t ldg, void* out, int tokens, int heads, int dv,
                                  float lambda, float scale, float eps, int dtype, cudaStream_t stream) {
    const int64_t items = (int64_t)tokens * heads;
    if (items <= 0) return 0;
    if (dv < 1) return ACORN_ERR_UNSUPPORTED;
    const int warps = 8;
    const uintptr_t align = dtype == ACORN_DTYPE_F32 ? 15 : 7;
    if (dv % 4 == 0 && dv <= 512 && ldg % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & align) == 0) {
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(diff_combine_vec_kernel<T>, dim3((unsigned)((items + warps - 1) / warps)),
                                                           dim3(32 * warps), 0, stream, (const T*)a, (const T*)g, ldg, (T*)out,
                                                           items, heads, dv, lambda, scale, eps));
    }
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(diff_combine_kernel<T>, dim3((unsigned)((items + warps - 1) / warps)),
                                                       dim3(32 * warps), 0, stream, (const T*)a, (const T*)g, ldg, (T*)out,
                                                       items, heads, dv, lambda, scale, eps));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- two float32 streams side by side, rounded
// out[t] = [a[t] | b[t]] in the activation dtype: the input of a product over both streams.
template <typename T>
__global__ void pair_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int64_t total,
                                 int H) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / (2 * H);
        const int c = (int)(i - t * 2 * H);
        out[i] = from_float<T>(c < H ? a[t * H + c] : b[t * H + c - H]);
    }
}

// widths that are multiples of four: four entries a thread
template <typename T>
__global__ void pair_rows_vec_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int64_t vecs,
                                     int H4) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / (2 * H4);
        const int c = (int)(i - t * 2 * H4);
        const float4 v = *reinterpret_cast<const float4*>((c < H4 ? a + (t * H4 + c) * 4 : b + (t * H4 + c - H4) * 4));
        Vec4<T>::store(out + i * 4, v);
    }
}

extern "C" int acorn_pair_rows(const float* a, const float* b, void* out, int tokens, int H, int dtype, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * 2 * H;
    if (total <= 0) return 0;
    if (H % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int64_t vecs = total / 4;
        int64_t vb = (vecs + 255) / 256;
        if (vb > 148 * 16) vb = 148 * 16;
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(pair_rows_vec_kernel<T>, dim3((int)vb), dim3(256), 0, stream, a, b,
                                                           (T*)out, vecs, H / 4));
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(pair_rows_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, a, b,
                                                       (T*)out, total, H));
    return ACORN_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- x[t, :] += row (float32): one vector added to every row
__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, int64_t total, int H) {
    pdl_wait();
    pdl_trigger();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        x[i] += row[i % H];
}

extern "C" int acorn_add_row(float* x, const float* row, int tokens, int H, cudaStream_t stream) {
    const int64_t total = (int64_t)tokens * H;
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return acorn_launch(add_row_kernel, dim3((int)blocks), dim3(256), 0, stream, x, row, total, H);
}
