// Small steps between matrix products: a clamped gated unit, norms of column segments, a matrix per
// head, and a constant on the logits.  All arithmetic is float32.
//
//   glu_clamp:     g = min(pg + bg, limit) ,  u = clamp(pu + bu, -limit, limit)
//                  out = g * sigmoid(alpha * g) * (u + offset)          pg, pu: columns f and F + f of one product
//   segment_norm:  for each segment (a run of columns of the input): y = x / sqrt(mean(x^2) + eps) * w
//                  (or y = x without a gain), written to one or two places
//   head_matmul:   y[n, h, :] = W_h x[n, h, :]  or  W_h^T x[n, h, :],  W_h = rows h*A .. h*A + A - 1 of W [H*A, B]
//   scale:         x *= c
//   latent_write:  per token: c = rmsnorm(latent) * w; the shared key part and every query head's first `dr`
//                  dims are turned by the token's position; the row [turned key part | c] goes into the key
//                  page and c into the value page (one head), the queries are turned in place
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

template <typename T>
__global__ void __launch_bounds__(256) glu_clamp_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                        const float* __restrict__ parts, int S, size_t part_stride,
                                                        const float* __restrict__ bias_g, const float* __restrict__ bias_u,
                                                        int F, size_t total, float limit, float alpha, float offset) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / F;
        const int f = (int)(i - n * F);
        const size_t at = n * 2 * F + f;
        float g = 0.f, u = 0.f;
        if (parts) {
            for (int s = 0; s < S; ++s) { g += parts[s * part_stride + at]; u += parts[s * part_stride + at + F]; }
        } else {
            g = to_float(in[at]);
            u = to_float(in[at + F]);
        }
        if (bias_g) g += bias_g[f];
        if (bias_u) u += bias_u[f];
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out[i] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + offset));
    }
}

// The same on a matrix (no partial sums) whose rows are whole 16-byte pieces: a thread takes 4 (float32) or 8
// (bfloat16) neighbouring units, gate and value in one 16-byte load each.
template <typename T>
__global__ void __launch_bounds__(256) glu_clamp_vec_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                            const float* __restrict__ bias_g, const float* __restrict__ bias_u,
                                                            int F, size_t packs, float limit, float alpha, float offset) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const int per_row = F / VEC;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < packs; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / per_row;
        const int f = (int)(i - n * per_row) * VEC;
        Vec16<T> gv, uv;
        gv.load(in + n * 2 * F + f);
        uv.load(in + n * 2 * F + F + f);
        __align__(16) T y[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float g = gv.get(e), u = uv.get(e);
            if (bias_g) g += bias_g[f + e];
            if (bias_u) u += bias_u[f + e];
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            y[e] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + offset));
        }
        *reinterpret_cast<uint4*>(out + n * F + f) = *reinterpret_cast<const uint4*>(y);
    }
}

__global__ void __launch_bounds__(256) scale_kernel(float* __restrict__ x, size_t total, float c) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] *= c;
}

constexpr int MAX_SEGMENTS = 4;

struct SegmentArgs {
    const void* x;             // [N, stride] in T
    long long stride;
    int count;
    int begin[MAX_SEGMENTS], len[MAX_SEGMENTS];
    const float* gain[MAX_SEGMENTS];           // null: the segment is copied
    void* dst0[MAX_SEGMENTS];                  // [N, dstride0] in T, written at column off0
    long long dstride0[MAX_SEGMENTS];
    int off0[MAX_SEGMENTS];
    void* dst1[MAX_SEGMENTS];                  // a second place, or null
    long long dstride1[MAX_SEGMENTS];
    int off1[MAX_SEGMENTS];
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(128) segment_norm_kernel(SegmentArgs a) {
    sb::pdl_launch_dependents();
    __shared__ float scratch[33];
    const int n = blockIdx.x, sg = blockIdx.y, len = a.len[sg];
    sb::pdl_wait();
    const T* x = (const T*)a.x + (size_t)n * a.stride + a.begin[sg];
    float rinv = 1.f;
    if (a.gain[sg]) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            const float v = to_float(x[i]);
            ss += v * v;
        }
        rinv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)len + a.eps);
    }
    T* d0 = (T*)a.dst0[sg] + (size_t)n * a.dstride0[sg] + a.off0[sg];
    T* d1 = a.dst1[sg] ? (T*)a.dst1[sg] + (size_t)n * a.dstride1[sg] + a.off1[sg] : nullptr;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float v = to_float(x[i]);
        const T y = a.gain[sg] ? from_float<T>(v * rinv * a.gain[sg][i]) : from_float<T>(v);
        d0[i] = y;
        if (d1) d1[i] = y;
    }
}

// A matrix per head.  A block serves one head, 16 tokens and 128 outputs; a thread owns an output and
// keeps 16 sums; the tokens' inputs sit in shared memory, four tokens side by side per input dim.
constexpr int HT = 16;
constexpr int HI = 128;        // input dims staged at a time

struct HeadArgs {
    const void* x; long long x_stride; int x_off, x_head;      // x[n, x_off + h * x_head + i]
    void* y; long long y_stride; int y_off, y_head;            // y[n, y_off + h * y_head + o]
    const void* w;                                             // [H*A, B] in T
    int A, B, transposed;      // 0: y = W_h x (A outputs, B inputs); 1: y = W_h^T x (B outputs, A inputs)
    int carry;                 // copy the `carry` values in front of every head's input to the front of its output
    int N;
};

template <typename T>
__global__ void __launch_bounds__(128) head_matmul_kernel(HeadArgs a) {
    sb::pdl_launch_dependents();
    __shared__ __align__(16) float xs[HI][HT];
    const int h = blockIdx.x, n0 = blockIdx.y * HT, o = blockIdx.z * 128 + threadIdx.x;
    const int nin = a.transposed ? a.A : a.B, nout = a.transposed ? a.B : a.A;
    const int nt = min(HT, a.N - n0);
    const T* w = (const T*)a.w + (size_t)h * a.A * a.B;
    sb::pdl_wait();
    const T* x = (const T*)a.x + (size_t)n0 * a.x_stride + a.x_off + (size_t)h * a.x_head;
    T* y = (T*)a.y + (size_t)n0 * a.y_stride + a.y_off + (size_t)h * a.y_head;
    if (blockIdx.z == 0 && a.carry > 0) {
        for (int i = threadIdx.x; i < nt * a.carry; i += blockDim.x) {
            const int t = i / a.carry, c = i - t * a.carry;
            y[(size_t)t * a.y_stride - a.carry + c] = x[(size_t)t * a.x_stride - a.carry + c];
        }
    }
    float acc[HT];
#pragma unroll
    for (int t = 0; t < HT; ++t) acc[t] = 0.f;
    for (int i0 = 0; i0 < nin; i0 += HI) {
        const int ni = min(HI, nin - i0);
        __syncthreads();
        for (int i = threadIdx.x; i < ni * HT; i += blockDim.x) {
            const int t = i / ni, d = i - t * ni;
            xs[d][t] = t < nt ? to_float(x[(size_t)t * a.x_stride + i0 + d]) : 0.f;
        }
        __syncthreads();
        if (o < nout) {
#pragma unroll 8
            for (int d = 0; d < ni; ++d) {
                const float wv = a.transposed ? to_float(w[(size_t)(i0 + d) * a.B + o]) : to_float(w[(size_t)o * a.B + i0 + d]);
#pragma unroll
                for (int t4 = 0; t4 < HT; t4 += 4) {
                    const float4 xv = *reinterpret_cast<const float4*>(&xs[d][t4]);
                    acc[t4] = fmaf(wv, xv.x, acc[t4]);
                    acc[t4 + 1] = fmaf(wv, xv.y, acc[t4 + 1]);
                    acc[t4 + 2] = fmaf(wv, xv.z, acc[t4 + 2]);
                    acc[t4 + 3] = fmaf(wv, xv.w, acc[t4 + 3]);
                }
            }
        }
    }
    if (o < nout) {
#pragma unroll
        for (int t = 0; t < HT; ++t)
            if (t < nt) y[(size_t)t * a.y_stride + o] = from_float<T>(acc[t]);
    }
}

struct LatentArgs {
    const void* down;          // [N, stride] in T: the latent at c_off (rank), the shared key part at r_off (dr)
    long long stride;
    int c_off, r_off, rank, dr;
    const float* gain;         // [rank]
    float eps;
    void* q;                   // [N, H*D] in T, D = dr + rank: every head's first dr dims are turned in place
    int H;
    const float* inv_freq;     // [dr / 2]
    int neighbours;            // 1: dim 2j turns with 2j + 1; 0: dim j with j + dr/2
    float magnitude;
    const int* positions;
    const int* token_rows;
    const int* block_table;
    int table_width, BS;
    void* k_pool;              // [pages, 1, BS, D]
    void* v_pool;              // [pages, 1, BS, rank]
};

template <typename T>
__global__ void __launch_bounds__(128) latent_write_kernel(LatentArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float cs[];           // dr/2 cosines, then dr/2 sines
    __shared__ float scratch[33];
    const int n = blockIdx.x, half = a.dr / 2, D = a.dr + a.rank;
    sb::pdl_wait();
    const int pos = a.positions[n];
    const int page = a.block_table[(size_t)a.token_rows[n] * a.table_width + pos / a.BS];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float ang = (float)pos * a.inv_freq[j];
        cs[j] = cosf(ang) * a.magnitude;
        cs[half + j] = sinf(ang) * a.magnitude;
    }
    const T* row = (const T*)a.down + (size_t)n * a.stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        const float v = to_float(row[a.c_off + i]);
        ss += v * v;
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)a.rank + a.eps);      // (its barriers also publish cs)
    const size_t slot = (size_t)page * a.BS + pos % a.BS;
    T* kr = (T*)a.k_pool + slot * D;
    T* vr = (T*)a.v_pool + slot * a.rank;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) {
        const T c = from_float<T>(to_float(row[a.c_off + i]) * rinv * a.gain[i]);
        kr[a.dr + i] = c;
        vr[i] = c;
    }
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const int ia = a.neighbours ? 2 * j : j, ib = a.neighbours ? 2 * j + 1 : j + half;
        const float u = to_float(row[a.r_off + ia]), v = to_float(row[a.r_off + ib]);
        kr[ia] = from_float<T>(u * cs[j] - v * cs[half + j]);
        kr[ib] = from_float<T>(v * cs[j] + u * cs[half + j]);
    }
    T* q = (T*)a.q + (size_t)n * a.H * D;
    for (int i = threadIdx.x; i < a.H * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const int ia = a.neighbours ? 2 * j : j, ib = a.neighbours ? 2 * j + 1 : j + half;
        T* qh = q + (size_t)h * D;
        const float u = to_float(qh[ia]), v = to_float(qh[ib]);
        qh[ia] = from_float<T>(u * cs[j] - v * cs[half + j]);
        qh[ib] = from_float<T>(v * cs[j] + u * cs[half + j]);
    }
}

inline int blocks_for(size_t total) { return (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8); }

}  // namespace

extern "C" int sb_glu_clamp(void* out, const void* in, const float* parts, int S, long long part_stride,
                            const float* bias_g, const float* bias_u, int N, int F, float limit, float alpha,
                            float offset, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && F > 0 && limit > 0.f, "glu_clamp: bad sizes N=%d F=%d or limit %f", N, F, limit);
    SB_REQUIRE((in != nullptr) != (parts != nullptr), "glu_clamp: one input, a matrix or partial sums");
    if (N == 0) return 0;
    const size_t total = (size_t)N * F;
    const int vec = dtype == SB_F32 ? 4 : 8;
    if (in != nullptr && F % vec == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const size_t packs = total / vec;
        if (dtype == SB_F32)
            sb::launch(glu_clamp_vec_kernel<float>, dim3(blocks_for(packs)), dim3(256), 0, stream, (float*)out, (const float*)in,
                       bias_g, bias_u, F, packs, limit, alpha, offset);
        else if (dtype == SB_BF16)
            sb::launch(glu_clamp_vec_kernel<__nv_bfloat16>, dim3(blocks_for(packs)), dim3(256), 0, stream, (__nv_bfloat16*)out,
                       (const __nv_bfloat16*)in, bias_g, bias_u, F, packs, limit, alpha, offset);
        else
            SB_REQUIRE(false, "glu_clamp: unknown dtype %d", dtype);
        SB_LAUNCH_CHECK();
    }
    if (dtype == SB_F32)
        sb::launch(glu_clamp_kernel<float>, dim3(blocks_for(total)), dim3(256), 0, stream, (float*)out, (const float*)in,
                   parts, S, (size_t)part_stride, bias_g, bias_u, F, total, limit, alpha, offset);
    else if (dtype == SB_BF16)
        sb::launch(glu_clamp_kernel<__nv_bfloat16>, dim3(blocks_for(total)), dim3(256), 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)in, parts, S, (size_t)part_stride, bias_g, bias_u, F, total, limit, alpha, offset);
    else
        SB_REQUIRE(false, "glu_clamp: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_scale(float* x, long long total, float c, cudaStream_t stream) {
    SB_REQUIRE(total >= 0, "scale: a negative size");
    if (total == 0) return 0;
    sb::launch(scale_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, stream, x, (size_t)total, c);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_segment_norm(const void* x, long long stride, int count, const int* begin, const int* len,
                               const void* const* gain, void* const* dst0, const long long* dstride0, const int* off0,
                               void* const* dst1, const long long* dstride1, const int* off1, float eps, int N,
                               int dtype, cudaStream_t stream) {
    SB_REQUIRE(count >= 1 && count <= MAX_SEGMENTS, "segment_norm: %d segments (1 to %d)", count, MAX_SEGMENTS);
    SB_REQUIRE(N >= 0 && N <= 2147483647 / 2, "segment_norm: bad token count %d", N);
    if (N == 0) return 0;
    SegmentArgs a;
    a.x = x; a.stride = stride; a.count = count; a.eps = eps;
    for (int i = 0; i < count; ++i) {
        SB_REQUIRE(len[i] > 0 && begin[i] >= 0 && dst0[i] != nullptr, "segment_norm: segment %d is empty or goes nowhere", i);
        a.begin[i] = begin[i]; a.len[i] = len[i]; a.gain[i] = (const float*)gain[i];
        a.dst0[i] = dst0[i]; a.dstride0[i] = dstride0[i]; a.off0[i] = off0[i];
        a.dst1[i] = dst1[i]; a.dstride1[i] = dstride1[i]; a.off1[i] = off1[i];
    }
    const dim3 grid(N, count);
    if (dtype == SB_F32) sb::launch(segment_norm_kernel<float>, grid, dim3(128), 0, stream, a);
    else if (dtype == SB_BF16) sb::launch(segment_norm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, a);
    else SB_REQUIRE(false, "segment_norm: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_head_matmul(void* y, long long y_stride, int y_off, int y_head, const void* x, long long x_stride,
                              int x_off, int x_head, const void* w, int H, int A, int B, int transposed, int carry,
                              int N, int dtype, cudaStream_t stream) {
    SB_REQUIRE(H > 0 && A > 0 && B > 0 && N >= 0 && carry >= 0, "head_matmul: bad sizes H=%d A=%d B=%d N=%d", H, A, B, N);
    SB_REQUIRE(carry <= x_off && carry <= y_off, "head_matmul: %d carried values do not fit in front of the heads", carry);
    if (N == 0) return 0;
    HeadArgs a;
    a.x = x; a.x_stride = x_stride; a.x_off = x_off; a.x_head = x_head; a.y = y; a.y_stride = y_stride;
    a.y_off = y_off; a.y_head = y_head; a.w = w; a.A = A; a.B = B; a.transposed = transposed; a.carry = carry; a.N = N;
    const int nout = transposed ? B : A;
    const dim3 grid(H, (N + HT - 1) / HT, (nout + 127) / 128);
    SB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "head_matmul: %d tokens exceed one launch", N);
    if (dtype == SB_F32) sb::launch(head_matmul_kernel<float>, grid, dim3(128), 0, stream, a);
    else if (dtype == SB_BF16) sb::launch(head_matmul_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, a);
    else SB_REQUIRE(false, "head_matmul: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_latent_write(const void* down, long long stride, int c_off, int r_off, int rank, int dr,
                               const float* gain, float eps, void* q, int H, const float* inv_freq, int neighbours,
                               float magnitude, const int* positions, const int* token_rows, const int* block_table,
                               int table_width, int page_size, void* k_pool, void* v_pool, int N, int dtype,
                               cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && H > 0 && rank > 0 && dr >= 0 && dr % 2 == 0, "latent_write: bad sizes H=%d rank=%d dr=%d", H, rank, dr);
    SB_REQUIRE(page_size > 0 && table_width > 0, "latent_write: bad page_size %d or table width %d", page_size, table_width);
    SB_REQUIRE(dr == 0 || inv_freq != nullptr, "latent_write: turning dims without a frequency table");
    if (N == 0) return 0;
    LatentArgs a;
    a.down = down; a.stride = stride; a.c_off = c_off; a.r_off = r_off; a.rank = rank; a.dr = dr; a.gain = gain;
    a.eps = eps; a.q = q; a.H = H; a.inv_freq = inv_freq; a.neighbours = neighbours; a.magnitude = magnitude;
    a.positions = positions; a.token_rows = token_rows; a.block_table = block_table; a.table_width = table_width;
    a.BS = page_size; a.k_pool = k_pool; a.v_pool = v_pool;
    const size_t smem = (size_t)(dr > 0 ? dr : 2) * sizeof(float);
    if (dtype == SB_F32) sb::launch(latent_write_kernel<float>, dim3(N), dim3(128), smem, stream, a);
    else if (dtype == SB_BF16) sb::launch(latent_write_kernel<__nv_bfloat16>, dim3(N), dim3(128), smem, stream, a);
    else SB_REQUIRE(false, "latent_write: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}
