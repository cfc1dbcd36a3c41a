// Per-head q/k RMSNorm + rotary position encoding + write of K and V into cache pages.
//
// qkv is the projection output [tokens, (nq + 2*nkv) * d]: nq query heads, then nkv
// key heads, then nkv value heads.  For every token and head, in float32:
//   q, k heads:  x <- x * rsqrt(mean(x^2) + eps) * w        (if a norm weight is given)
//                rotate the first `rot` dims by angle pos * inv_freq[j]:
//                  pairing 0 (half):        (x[j], x[j + rot/2])
//                  pairing 1 (interleaved): (x[2j], x[2j+1])
//                  (a, b) <- (a cos - b sin, b cos + a sin)
//   q is written back in place; k goes to the K page, v (untouched) to the V page.
// Cache layout per layer: [num_pages, nkv, page_size, d]; the token at position p of
// row r lives in page block_table[r * table_stride + p / P - page_base[r]], slot p % P.
// `magnitude` multiplies cos and sin (position encodings with stretched frequencies).  With norm_after the
// order is the other way round: the head is rotated first and then brought to unit root mean square,
// x <- x * rsqrt(mean(x^2) + eps) over rotated and unrotated entries alike (times w if a weight is given,
// no weight otherwise); both are the general kernel's.
// With write_kv = 0 only the query heads are processed (a layer that reads another
// layer's cache).  Value heads may have a width of their own (dv; their pages then hold rows of dv),
// a row of qkv may be wider than its heads (ld elements), and with v_from_k the values are the keys as
// projected, before norm and rotation: the row then holds no value heads, [q | k] only.
//
// Before all that, optionally, a bias per channel and a short causal convolution over time on every
// channel of q, k and v (conv_w [channels, taps], the last tap for the current token):
//   u_t = row_t + bias;   x_t = sum_j conv_w[:, j] * u_(t - taps + 1 + j)
// with the u before a step's first token taken from the request's state slot (the last taps - 1 of
// them, [taps - 1, channels] float32 in time order, zeros when the request starts; kept up to date by
// conv_state_update with the same bias).  A token's convolution reads its neighbours' rows as projected,
// so the queries then go to a buffer of their own (q_out) instead of back into qkv.
#include "common.cuh"

#define QK_MAX_TAPS 16

struct QkConv {
    const float* w;           // [channels, taps] or null: no convolution
    const float* bias;        // [channels] or null
    float* state;             // [slots, slot_stride] float32
    int64_t slot_stride, conv_off;
    const int* row_start;
    const int* row_slot;
    int taps;                 // >= 1 when w is given
    int channels;             // nq d + nkv d + nkv dv
    int update_single;        // a row of a single token shifts its own memory here (conv_state_update then skips such rows)
};

template <typename T>
__global__ void qk_rope_kv_kernel(T* __restrict__ qkv, const float* __restrict__ q_w,
                                  const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                                  const int* __restrict__ positions, const int* __restrict__ token_row,
                                  const int* __restrict__ block_table, const int* __restrict__ page_base,
                                  int table_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                  int tokens, int nq, int nkv, int d, int rot, int pairing, int P,
                                  float eps, int write_kv, int64_t ld, int dv, int v_from_k, QkConv cv,
                                  T* __restrict__ q_out, int64_t ld_q, float magnitude, int norm_after) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_trigger();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t item = (int64_t)blockIdx.x * warps_per_block + warp;
    if (item >= (int64_t)tokens * heads) return;
    const int t = (int)(item / heads);
    const int h = (int)(item - (int64_t)t * heads);
    float* x = smem + warp * d;
    T* src = qkv + (int64_t)t * ld + (int64_t)h * d;
    const int pos = positions[t];

    T* dst = q_out ? q_out + (int64_t)t * ld_q + (int64_t)h * d : src;   // q: in place unless a buffer is given
    int64_t chan = (int64_t)h * d;                                        // first channel of this head in a row
    if (h >= nq) {
        const int r = token_row[t];
        const int kvh = (h - nq) % nkv;
        const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
        const int64_t slot = ((int64_t)page * nkv + kvh) * P + (pos % P);
        dst = (h < nq + nkv) ? k_pages + slot * d : v_pages + slot * dv;
        if (h >= nq + nkv) {    // the value head's source: its own columns, or the key head as projected
            chan = v_from_k ? (int64_t)(nq + kvh) * d : (int64_t)(nq + nkv) * d + (int64_t)kvh * dv;
            src = qkv + (int64_t)t * ld + chan;
        }
    }
    // element i of this head after bias and convolution (the plain element without them)
    int i0 = 0;
    float* cstate = nullptr;
    bool shift = false;
    if (cv.w) {
        const int r = token_row[t];
        i0 = t - cv.row_start[r];                                         // the token's index within its row
        if (cv.taps > 1) cstate = cv.state + (int64_t)cv.row_slot[r] * cv.slot_stride + cv.conv_off;
        shift = cv.update_single && cv.taps > 1 && cv.row_start[r + 1] - cv.row_start[r] == 1;
    }
    auto element = [&](int i) -> float {
        const float own = to_float(src[i]) + (cv.bias ? cv.bias[chan + i] : 0.f);
        if (!cv.w) return own;
        const float* w = cv.w + (chan + i) * cv.taps;
        float acc = 0.f;
        for (int j = 0; j < cv.taps - 1; ++j) {
            const int idx = i0 - (cv.taps - 1) + j;                       // input index within the row; negative: before the step
            const float in = idx >= 0 ? to_float(src[(int64_t)(idx - i0) * ld + i]) + (cv.bias ? cv.bias[chan + i] : 0.f)
                                      : cstate[(int64_t)(cv.taps - 1 + idx) * cv.channels + chan + i];
            acc = fmaf(w[j], in, acc);
            // the row's only token: a channel is read and written by this thread alone, oldest entry first
            if (shift && j > 0) cstate[(int64_t)(j - 1) * cv.channels + chan + i] = in;
        }
        if (shift) cstate[(int64_t)(cv.taps - 2) * cv.channels + chan + i] = own;
        return fmaf(w[cv.taps - 1], own, acc);
    };
    if (h >= nq + nkv) {   // value head: copy
        if (cv.w || cv.bias) {
            for (int i = lane; i < dv; i += 32) dst[i] = from_float<T>(element(i));
        } else {
            for (int i = lane; i < dv; i += 32) dst[i] = src[i];
        }
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float v = element(i);
        x[i] = v;
        ss += v * v;
    }
    const float* w = (h < nq) ? q_w : k_w;
    if (w && !norm_after) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + eps);
        __syncwarp();
        for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * w[i];
    }
    __syncwarp();
    const int half = rot >> 1;
    if (norm_after) {
        // the rotation first (cos and sin times `magnitude`), then the head brought to unit root mean square
        // (times the weight, if one is given): the rotated part's length depends on the magnitude
        float ss2 = 0.f;
        for (int j = lane; j < half; j += 32) {
            const int ia = pairing == 0 ? j : 2 * j;
            const int ib = pairing == 0 ? j + half : 2 * j + 1;
            float s, c;
            sincosf((float)pos * inv_freq[j], &s, &c);
            s *= magnitude;
            c *= magnitude;
            const float a = x[ia], b = x[ib];
            const float ra = a * c - b * s, rb = b * c + a * s;
            x[ia] = ra;
            x[ib] = rb;
            ss2 += ra * ra + rb * rb;
        }
        for (int i = rot + lane; i < d; i += 32) ss2 += x[i] * x[i];
        ss2 = warp_sum(ss2);
        const float inv = rsqrtf(ss2 / (float)d + eps);
        __syncwarp();
        for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(x[i] * inv * (w ? w[i] : 1.f));
        return;
    }
    for (int j = lane; j < half; j += 32) {
        const int ia = pairing == 0 ? j : 2 * j;
        const int ib = pairing == 0 ? j + half : 2 * j + 1;
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        s *= magnitude;
        c *= magnitude;
        const float a = x[ia], b = x[ib];
        dst[ia] = from_float<T>(a * c - b * s);
        dst[ib] = from_float<T>(b * c + a * s);
    }
    for (int i = rot + lane; i < d; i += 32) dst[i] = from_float<T>(x[i]);
}

// Rotation of neighbouring pairs, then the norm (norm_after), for heads of up to 128 entries that are multiples of four:
// a warp a (token, head), four consecutive entries a lane (8- or 16-byte accesses), which are two whole pairs, so that
// rotation, sum of squares and write need neither shared memory nor a second pass.  Value heads are the key heads as
// projected (v_from_k) or columns of their own.
template <typename T>
__global__ void qk_rope_norm_after_vec_kernel(T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                              const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                              const int* __restrict__ token_row, const int* __restrict__ block_table,
                                              const int* __restrict__ page_base, int table_stride, T* __restrict__ k_pages,
                                              T* __restrict__ v_pages, int tokens, int nq, int nkv, int d, int rot, int P,
                                              float eps, int write_kv, int64_t ld, int v_from_k, float magnitude) {
    pdl_wait();
    pdl_trigger();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t item = (int64_t)blockIdx.x * warps_per_block + warp;
    if (item >= (int64_t)tokens * heads) return;
    const int t = (int)(item / heads);
    const int h = (int)(item - (int64_t)t * heads);
    const int pos = positions[t];
    const int i = 4 * lane;                                              // this lane's first entry
    const bool live = i < d;
    const T* src = qkv + (int64_t)t * ld + (int64_t)h * d;
    T* dst = qkv + (int64_t)t * ld + (int64_t)h * d;                     // q: in place
    if (h >= nq) {
        const int r = token_row[t];
        const int kvh = (h - nq) % nkv;
        const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
        const int64_t slot = ((int64_t)page * nkv + kvh) * P + (pos % P);
        dst = ((h < nq + nkv) ? k_pages : v_pages) + slot * d;
        if (h >= nq + nkv) src = qkv + (int64_t)t * ld + (v_from_k ? (int64_t)(nq + kvh) * d : (int64_t)(nq + nkv + kvh) * d);
    }
    float4 x = live ? Vec4<T>::load(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (h >= nq + nkv) {                                                 // a value head: as projected
        if (live) Vec4<T>::store(dst + i, x);
        return;
    }
    if (live && i < rot) {                                               // pairs (i, i + 1) and, if rotated too, (i + 2, i + 3)
        float sn, cs;
        sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float a = x.x, b = x.y;
        x.x = a * cs - b * sn;
        x.y = b * cs + a * sn;
        if (i + 2 < rot) {
            sincosf((float)pos * inv_freq[(i >> 1) + 1], &sn, &cs);
            sn *= magnitude;
            cs *= magnitude;
            const float c = x.z, e = x.w;
            x.z = c * cs - e * sn;
            x.w = e * cs + c * sn;
        }
    }
    const float ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
    const float inv = rsqrtf(ss / (float)d + eps);
    const float* w = (h < nq) ? q_w : k_w;
    if (live) {
        const float4 wv = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        Vec4<T>::store(dst + i, make_float4(x.x * inv * wv.x, x.y * inv * wv.y, x.z * inv * wv.z, x.w * inv * wv.w));
    }
}

// The same for the common case (whole head rotated, half pairing, head size 16, 32, 64, 128 or
// 256): a group of d / 8 lanes takes ROPE_HPG consecutive heads of one token, each lane holding
// four rotary pairs (x[4l .. 4l+3], x[d/2 + 4l .. d/2 + 4l+3]) of every head in registers; vector
// loads (all heads first, then the arithmetic) and stores, no shared memory.  The angles depend
// on the token and the lane only, so cos and sin are computed once for the heads of a group.
// ROPE_HPG = 4 for many tokens (fewer sincos), 1 for few (a decode step: more threads, shorter chains).
template <typename T, int G, int ROPE_HPG>
__global__ void qk_rope_kv_vec_kernel(T* __restrict__ qkv, const float* __restrict__ q_w,
                                      const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                                      const int* __restrict__ positions, const int* __restrict__ token_row,
                                      const int* __restrict__ block_table, const int* __restrict__ page_base,
                                      int table_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                      int tokens, int nq, int nkv, int P, float eps, int write_kv) {
    constexpr int D = G * 8, HALF = D / 2;
    pdl_wait();
    pdl_trigger();
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int groups = (heads + ROPE_HPG - 1) / ROPE_HPG;                // head groups per token
    const int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int l = threadIdx.x % G;
    const bool active = item < (int64_t)tokens * groups;
    const int64_t it = active ? item : 0;
    const int t = (int)(it / groups);
    const int h0 = (int)(it - (int64_t)t * groups) * ROPE_HPG;
    T* tok = qkv + (int64_t)t * (nq + 2 * nkv) * D;
    const int pos = positions[t];
    float4 a[ROPE_HPG], b[ROPE_HPG];
#pragma unroll
    for (int i = 0; i < ROPE_HPG; ++i) {
        const int h = min(h0 + i, heads - 1);
        a[i] = Vec4<T>::load(tok + (int64_t)h * D + 4 * l);
        b[i] = Vec4<T>::load(tok + (int64_t)h * D + HALF + 4 * l);
    }
    int64_t page_off = 0;                                                // of this token's slot, in rows of D
    if (h0 + ROPE_HPG > nq && write_kv) {
        const int r = token_row[t];
        const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
        page_off = (int64_t)page * nkv * P + (pos % P);
    }
    float s0 = 0.f, c0 = 1.f, s1 = 0.f, c1 = 1.f, s2 = 0.f, c2 = 1.f, s3 = 0.f, c3 = 1.f;
    if (h0 < nq + nkv) {
        const float4 f = *reinterpret_cast<const float4*>(inv_freq + 4 * l);
        sincosf((float)pos * f.x, &s0, &c0);
        sincosf((float)pos * f.y, &s1, &c1);
        sincosf((float)pos * f.z, &s2, &c2);
        sincosf((float)pos * f.w, &s3, &c3);
    }
#pragma unroll
    for (int i = 0; i < ROPE_HPG; ++i) {
        const bool valid = active && h0 + i < heads;
        const int h = min(h0 + i, heads - 1);
        float4 x = a[i], y = b[i];
        T* dst = tok + (int64_t)h * D;                                   // q: in place
        if (h >= nq) {
            const int kvh = (h - nq) % nkv;
            dst = ((h < nq + nkv) ? k_pages : v_pages) + (page_off + (int64_t)kvh * P) * D;
        }
        // the sum of squares is reduced by every lane of the warp, whatever its head is: lanes of
        // one warp hold heads of different kinds
        float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w + y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (h < nq + nkv) {
            const float* w = (h < nq) ? q_w : k_w;
            if (w) {
                const float inv = rsqrtf(ss / (float)D + eps);
                const float4 wa = *reinterpret_cast<const float4*>(w + 4 * l);
                const float4 wb = *reinterpret_cast<const float4*>(w + HALF + 4 * l);
                x = make_float4(x.x * inv * wa.x, x.y * inv * wa.y, x.z * inv * wa.z, x.w * inv * wa.w);
                y = make_float4(y.x * inv * wb.x, y.y * inv * wb.y, y.z * inv * wb.z, y.w * inv * wb.w);
            }
            const float4 ra = make_float4(x.x * c0 - y.x * s0, x.y * c1 - y.y * s1, x.z * c2 - y.z * s2, x.w * c3 - y.w * s3);
            const float4 rb = make_float4(y.x * c0 + x.x * s0, y.y * c1 + x.y * s1, y.z * c2 + x.z * s2, y.w * c3 + x.w * s3);
            x = ra;
            y = rb;
        }
        if (valid) {
            Vec4<T>::store(dst + 4 * l, x);
            Vec4<T>::store(dst + HALF + 4 * l, y);
        }
    }
}

template <typename T, int G, int ROPE_HPG>
static int launch_rope_vec_hpg(T* qkv, const float* q_w, const float* k_w, const float* inv_freq, const int* positions,
                           const int* token_row, const int* block_table, const int* page_base, int table_stride,
                           T* k_pages, T* v_pages, int tokens, int nq, int nkv, int P, float eps, int write_kv,
                           cudaStream_t stream) {
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t threads = (int64_t)tokens * ((heads + ROPE_HPG - 1) / ROPE_HPG) * G;
    const int64_t blocks = (threads + 255) / 256;
    return acorn_launch(qk_rope_kv_vec_kernel<T, G, ROPE_HPG>, dim3((unsigned)blocks), dim3(256), 0, stream, qkv, q_w,
                        k_w, inv_freq, positions, token_row, block_table, page_base, table_stride, k_pages, v_pages,
                        tokens, nq, nkv, P, eps, write_kv);
}

template <typename T, int G>
static int launch_rope_vec(T* qkv, const float* q_w, const float* k_w, const float* inv_freq, const int* positions,
                           const int* token_row, const int* block_table, const int* page_base, int table_stride,
                           T* k_pages, T* v_pages, int tokens, int nq, int nkv, int P, float eps, int write_kv,
                           cudaStream_t stream) {
    if (tokens > 256)
        return launch_rope_vec_hpg<T, G, 4>(qkv, q_w, k_w, inv_freq, positions, token_row, block_table, page_base,
                                            table_stride, k_pages, v_pages, tokens, nq, nkv, P, eps, write_kv, stream);
    return launch_rope_vec_hpg<T, G, 1>(qkv, q_w, k_w, inv_freq, positions, token_row, block_table, page_base,
                                        table_stride, k_pages, v_pages, tokens, nq, nkv, P, eps, write_kv, stream);
}

// Bias, convolution over time, norm and cache write for heads that are not rotated, four channels a lane
// (8- or 16-byte accesses): LPH lanes a head (a power of two, at most 32, 4 LPH >= the wider of d and dv),
// a lane's weights of all taps in registers (TAPS of them, 0: no convolution), the taps in the order of the
// general kernel.  A lane walks tpt consecutive tokens of the step and carries the inputs before the current
// token along in registers while it stays within a row (a row's first token reads them from the request's
// memory).  Widths, row strides and state offsets are multiples of four.
template <typename T, int TAPS>
__global__ void qk_conv_kv_vec_kernel(T* __restrict__ qkv, const float* __restrict__ q_w,
                                      const float* __restrict__ k_w, const int* __restrict__ positions,
                                      const int* __restrict__ token_row, const int* __restrict__ block_table,
                                      const int* __restrict__ page_base, int table_stride, T* __restrict__ k_pages,
                                      T* __restrict__ v_pages, int tokens, int nq, int nkv, int d, int dv, int P,
                                      float eps, int write_kv, int64_t ld, QkConv cv, T* __restrict__ q_out,
                                      int64_t ld_q, int lph_log2, int tpt) {
    pdl_wait();
    pdl_trigger();
    constexpr int PAST = TAPS > 1 ? TAPS - 1 : 1;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t item = gid >> lph_log2;
    const int l = (int)(gid & ((1 << lph_log2) - 1));
    const int64_t chunks = ((int64_t)tokens + tpt - 1) / tpt;
    const bool in_range = item < chunks * heads;
    const int64_t it = in_range ? item : 0;
    const int64_t t_first = (it / heads) * tpt;
    const int h = (int)(it % heads);
    const bool is_v = h >= nq + nkv;
    const bool lane_on = in_range && 4 * l < (is_v ? dv : d);
    const int64_t chan = (is_v ? (int64_t)(nq + nkv) * d + (int64_t)(h - nq - nkv) * dv : (int64_t)h * d) + 4 * l;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 b = zero, g = zero;
    const float* nw = is_v ? nullptr : (h < nq ? q_w : k_w);
    float w[TAPS > 0 ? 4 * TAPS : 1];                                     // w[i * TAPS + j]: channel i of the lane, tap j
    if (lane_on) {
        if (cv.bias) b = *reinterpret_cast<const float4*>(cv.bias + chan);
        if (nw) g = *reinterpret_cast<const float4*>(nw + 4 * l);
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const float4 v = *reinterpret_cast<const float4*>(cv.w + chan * TAPS + 4 * j);
            w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
    }
    float4 past[PAST];                                                    // the inputs before the current token, oldest first
    float4 before = zero;                                                 // the token before's own input
    for (int k = 0; k < tpt; ++k) {
        const int64_t t = t_first + k;
        const bool active = lane_on && t < tokens;
        float4 x = zero;
        int r = 0;
        if (active) {
            T* src = qkv + t * ld + chan;
            const float4 raw = Vec4<T>::load(src);
            const float4 own = make_float4(raw.x + b.x, raw.y + b.y, raw.z + b.z, raw.w + b.w);
            r = token_row[t];
            if constexpr (TAPS == 0) {
                x = own;
            } else {
                if constexpr (TAPS > 1) {
                    const int i0 = (int)t - cv.row_start[r];              // the token's index within its row
                    if (k == 0 || i0 == 0) {
                        float* cstate = cv.state + (int64_t)cv.row_slot[r] * cv.slot_stride + cv.conv_off + chan;
                        const bool shift = cv.update_single && cv.row_start[r + 1] - cv.row_start[r] == 1;
#pragma unroll
                        for (int j = 0; j < TAPS - 1; ++j) {
                            const int idx = i0 - (TAPS - 1) + j;          // negative: before the step
                            if (idx >= 0) {
                                const float4 u = Vec4<T>::load(src + (int64_t)(idx - i0) * ld);
                                past[j] = make_float4(u.x + b.x, u.y + b.y, u.z + b.z, u.w + b.w);
                            } else {
                                past[j] = *reinterpret_cast<const float4*>(cstate + (int64_t)(TAPS - 1 + idx) * cv.channels);
                            }
                            // the row's only token: a lane alone reads and writes its channels, oldest entry first
                            if (shift && j > 0) *reinterpret_cast<float4*>(cstate + (int64_t)(j - 1) * cv.channels) = past[j];
                        }
                        if (shift) *reinterpret_cast<float4*>(cstate + (int64_t)(TAPS - 2) * cv.channels) = own;
                    } else {
#pragma unroll
                        for (int j = 0; j < TAPS - 2; ++j) past[j] = past[j + 1];
                        past[TAPS - 2] = before;
                    }
#pragma unroll
                    for (int j = 0; j < TAPS - 1; ++j) {
                        x.x = fmaf(w[j], past[j].x, x.x);
                        x.y = fmaf(w[TAPS + j], past[j].y, x.y);
                        x.z = fmaf(w[2 * TAPS + j], past[j].z, x.z);
                        x.w = fmaf(w[3 * TAPS + j], past[j].w, x.w);
                    }
                }
                x.x = fmaf(w[TAPS - 1], own.x, x.x);
                x.y = fmaf(w[2 * TAPS - 1], own.y, x.y);
                x.z = fmaf(w[3 * TAPS - 1], own.z, x.z);
                x.w = fmaf(w[4 * TAPS - 1], own.w, x.w);
            }
            before = own;
        }
        // every lane of the warp takes part in the sums, whatever its head is
        float ss = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        for (int o = (1 << lph_log2) >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (active) {
            if (nw) {
                const float inv = rsqrtf(ss / (float)d + eps);
                x = make_float4(x.x * inv * g.x, x.y * inv * g.y, x.z * inv * g.z, x.w * inv * g.w);
            }
            T* dst;
            if (h < nq) {
                dst = q_out ? q_out + t * ld_q + chan : qkv + t * ld + chan;
            } else {
                const int pos = positions[t];
                const int kvh = (h - nq) % nkv;
                const int page = block_table[(int64_t)r * table_stride + (pos / P - page_base[r])];
                const int64_t slot = ((int64_t)page * nkv + kvh) * P + (pos % P);
                dst = (is_v ? v_pages + slot * dv : k_pages + slot * d) + 4 * l;
            }
            Vec4<T>::store(dst, x);
        }
    }
}

template <typename T, int TAPS>
static int launch_conv_vec(T* qkv, const float* q_w, const float* k_w, const int* positions, const int* token_row,
                           const int* block_table, const int* page_base, int table_stride, T* k_pages, T* v_pages,
                           int tokens, int nq, int nkv, int d, int dv, int P, float eps, int write_kv, int64_t ld,
                           const QkConv& cv, T* q_out, int64_t ld_q, cudaStream_t stream) {
    const int widest = (write_kv && dv > d) ? dv : d;
    int lph_log2 = 0;
    while ((4 << lph_log2) < widest) ++lph_log2;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int tpt = tokens > 1024 ? 8 : (tokens > 256 ? 4 : 1);                // a step of few tokens: a lane a token
    const int64_t threads = (((int64_t)tokens + tpt - 1) / tpt * heads) << lph_log2;
    const int block = threads >= 256 ? 256 : 128;
    return acorn_launch(qk_conv_kv_vec_kernel<T, TAPS>, dim3((unsigned)((threads + block - 1) / block)), dim3(block), 0,
                        stream, qkv, q_w, k_w, positions, token_row, block_table, page_base, table_stride, k_pages,
                        v_pages, tokens, nq, nkv, d, dv, P, eps, write_kv, ld, cv, q_out, ld_q, lph_log2, tpt);
}

static bool qk_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int acorn_qk_rope_kv(void* qkv, const float* q_w, const float* k_w, const float* inv_freq,
                                const int* positions, const int* token_row, const int* block_table,
                                const int* page_base, int table_stride, void* k_pages, void* v_pages,
                                int tokens, int nq, int nkv, int d, int rot, int pairing, int P,
                                float eps, int write_kv, int dtype, int64_t ld, int dv, int v_from_k,
                                const float* conv_w, int taps, const float* bias, float* state,
                                int64_t slot_stride, int64_t conv_off, const int* row_start, const int* row_slot,
                                void* q_out, int64_t ld_q, int update_single, float magnitude, int norm_after,
                                cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d > 1024 || rot > d || (rot & 1) || dv < 1 || dv > 1024 || (v_from_k && dv != d)) return ACORN_ERR_UNSUPPORTED;
    QkConv cv;
    cv.w = conv_w; cv.bias = bias; cv.state = state; cv.slot_stride = slot_stride; cv.conv_off = conv_off;
    cv.row_start = row_start; cv.row_slot = row_slot; cv.taps = taps; cv.update_single = update_single;
    cv.channels = (nq + nkv) * d + (v_from_k ? 0 : nkv * dv);
    if (conv_w && (taps < 1 || taps > QK_MAX_TAPS || v_from_k || q_out == nullptr || row_start == nullptr ||
                   (taps > 1 && (state == nullptr || row_slot == nullptr))))
        return ACORN_ERR_UNSUPPORTED;
    const bool special = magnitude != 1.f || norm_after;            // the general kernel alone knows these
    const bool plain_rows = conv_w == nullptr && bias == nullptr && q_out == nullptr;
    if (plain_rows && !special && rot == d && pairing == 0 && dv == d && !v_from_k && ld == (int64_t)(nq + 2 * nkv) * d &&
        (d == 16 || d == 32 || d == 64 || d == 128 || d == 256)) {
#define ROPE_VEC(G)                                                                                                  \
    ACORN_DISPATCH_DTYPE(dtype, T, return (launch_rope_vec<T, G>((T*)qkv, q_w, k_w, inv_freq, positions, token_row,   \
                                                                  block_table, page_base, table_stride, (T*)k_pages,   \
                                                                  (T*)v_pages, tokens, nq, nkv, P, eps, write_kv,      \
                                                                  stream)))
        switch (d) {
            case 16: ROPE_VEC(2); break;
            case 32: ROPE_VEC(4); break;
            case 64: ROPE_VEC(8); break;
            case 128: ROPE_VEC(16); break;
            default: ROPE_VEC(32); break;
        }
#undef ROPE_VEC
    }
    if (plain_rows && norm_after && pairing == 1 && d % 4 == 0 && d <= 128 && dv == d && ld % 4 == 0 && qk_aligned16(qkv) &&
        qk_aligned16(k_pages) && qk_aligned16(v_pages) && qk_aligned16(q_w) && qk_aligned16(k_w)) {
        const int warps = 4;
        const int64_t items = (int64_t)tokens * (write_kv ? (nq + 2 * nkv) : nq);
        ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(
            qk_rope_norm_after_vec_kernel<T>, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream,
            (T*)qkv, q_w, k_w, inv_freq, positions, token_row, block_table, page_base, table_stride, (T*)k_pages,
            (T*)v_pages, tokens, nq, nkv, d, rot, P, eps, write_kv, ld, v_from_k, magnitude));
    }
    const int vec_taps = conv_w ? taps : 0;
    if (!plain_rows && !special && rot == 0 && !v_from_k && vec_taps <= 4 && d % 4 == 0 && dv % 4 == 0 && d <= 128 && dv <= 128 &&
        ld % 4 == 0 && ld_q % 4 == 0 && slot_stride % 4 == 0 && conv_off % 4 == 0 && qk_aligned16(qkv) &&
        qk_aligned16(q_out) && qk_aligned16(k_pages) && qk_aligned16(v_pages) && qk_aligned16(q_w) &&
        qk_aligned16(k_w) && qk_aligned16(conv_w) && qk_aligned16(bias) && qk_aligned16(state)) {
#define CONV_VEC(TAPS)                                                                                                \
    ACORN_DISPATCH_DTYPE(dtype, T, return (launch_conv_vec<T, TAPS>((T*)qkv, q_w, k_w, positions, token_row,           \
                                                                     block_table, page_base, table_stride, (T*)k_pages, \
                                                                     (T*)v_pages, tokens, nq, nkv, d, dv, P, eps,       \
                                                                     write_kv, ld, cv, (T*)q_out, ld_q, stream)))
        switch (vec_taps) {
            case 0: CONV_VEC(0); break;
            case 1: CONV_VEC(1); break;
            case 2: CONV_VEC(2); break;
            case 3: CONV_VEC(3); break;
            default: CONV_VEC(4); break;
        }
#undef CONV_VEC
    }
    const int warps = 4;
    const int heads = write_kv ? (nq + 2 * nkv) : nq;
    const int64_t items = (int64_t)tokens * heads;
    const int64_t blocks = (items + warps - 1) / warps;
    const size_t smem = (size_t)warps * d * sizeof(float);
    ACORN_DISPATCH_DTYPE(dtype, T, return acorn_launch(
        qk_rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream, (T*)qkv, q_w, k_w, inv_freq,
        positions, token_row, block_table, page_base, table_stride, (T*)k_pages, (T*)v_pages, tokens, nq, nkv, d, rot,
        pairing, P, eps, write_kv, ld, dv, v_from_k, cv, (T*)q_out, ld_q, magnitude, norm_after));
    return ACORN_ERR_UNSUPPORTED;
}

// cos and sin of position * inv_freq[j] for every token of a step: out[t][j] = cos, out[t][half + j] = sin
// (float32, the accurate sincosf).  One table serves every layer of the step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ out, int tokens, int half) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)tokens * half) return;
    const int t = (int)(i / half), j = (int)(i - (int64_t)t * half);
    float s, c;
    sincosf((float)positions[t] * inv_freq[j], &s, &c);
    out[(int64_t)t * 2 * half + j] = c;
    out[(int64_t)t * 2 * half + half + j] = s;
}

extern "C" int acorn_rope_table(const int* positions, const float* inv_freq, float* out, int tokens, int half,
                                cudaStream_t stream) {
    if (tokens <= 0 || half <= 0) return 0;
    const int64_t n = (int64_t)tokens * half;
    return acorn_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, positions, inv_freq,
                        out, tokens, half);
}
