// The residual as several streams (hyper-connections), folded and normed in one pass.
//
// A row holds `s` streams x_1 .. x_s of d floats (s = 1: the ordinary residual).  A sublayer reads
// u = sum_t in[t] x_t, and its output y joins all streams at once:
//     x_t <- sum_f mix[f][t] x_f + mult * outw[t] * y
// The kernel does, per row, whatever of this is waiting, then norms the next reading:
//     y   = scale_a * (sum_p A[p] + bias) + scale_b * sum_p B[p]      (two branches' partial sums, B optional)
//     x_t <- sum_f mix[f][t] x_f + mult * outw[t] * y                 (mix null: identity; outw null: ones)
//     u   = sum_t in[t] x_t                                           (in null: ones, the plain sum)
//     out = (u - mean(u)) / sqrt(mean((u - mean)^2) + eps) * gain     (center = 1: layer norm)
//     out = u / sqrt(mean(u^2) + eps) * gain                          (center = 0: RMS norm)
//     out = u                                                         (gain null)
// With `init` the streams do not exist yet: every x_t starts as init[row].  With `row_index` only
// the named rows are read and nothing is written back (the rows whose logits are wanted).
// Everything is float32; the variance is taken over the deviations in a second pass over the row,
// which sits in shared memory.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

constexpr int SMAX = 8;

struct HyperArgs {
    float* streams;            // [rows, s, d]
    const float* init;         // [rows, d] or null
    const float* a; int SA; size_t stride_a; float scale_a;
    const float* b; int SB; size_t stride_b; float scale_b;
    const float* bias;         // [d] or null
    const float* mix;          // [s, s] (from, to) or null
    const float* outw;         // [s] or null
    const float* inw;          // [s] or null
    const float* gain;         // [d] or null
    float mult, eps;
    int center;
    void* out;                 // [M, d] or null
    float* read_out;           // [M, d] float32 or null: u itself
    const int* row_index;
    int s, d, write_streams, has_branch;
};

// E consecutive columns a thread and step: 4 (16-byte accesses; d a multiple of 4 and aligned rows) or 1.
// Everything a column needs (its streams, every partial sum of both branches, the bias) is loaded before
// anything is added, so a row costs one or two round trips to memory however many streams and parts there are.
template <int E> struct Pack;
template <> struct Pack<1> {
    float v[1];
    __device__ __forceinline__ void load(const float* p) { v[0] = __ldg(p); }
    __device__ __forceinline__ void load_rw(const float* p) { v[0] = *p; }
    __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <> struct Pack<4> {
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void load_rw(const float* p) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};

// SM_: most streams the instance takes; PA, PB: partial sums of the first and second branch whose loads are in
// flight at once (more are added one by one afterwards).
template <typename T, int E, int SM_, int PA, int PB>
__global__ void __launch_bounds__(E == 4 ? 256 : 1024) hyper_fold_norm_kernel(HyperArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ __align__(16) float urow[];         // d floats
    __shared__ float scratch[33];
    __shared__ float c_mix[SMAX * SMAX], c_out[SMAX], c_in[SMAX];
    const int s = a.s, d = a.d, m = blockIdx.x;
    // constants of the model: they may be read before the kernel before this one has finished
    for (int i = threadIdx.x; i < s * s; i += blockDim.x) c_mix[i] = a.mix ? a.mix[i] : (i / s == i % s ? 1.f : 0.f);
    for (int i = threadIdx.x; i < s; i += blockDim.x) {
        c_out[i] = (a.outw ? a.outw[i] : 1.f) * a.mult;
        c_in[i] = a.inw ? a.inw[i] : 1.f;
    }
    sb::pdl_wait();
    __syncthreads();
    const int r = a.row_index ? a.row_index[m] : m;
    float* xs = a.streams + (size_t)r * s * d;
    float total = 0.f;
    for (int i = threadIdx.x * E; i < d; i += blockDim.x * E) {
        Pack<E> x[SM_], pa[PA], pb[PB], bias;
        // ---- every load of the column first
        if (a.init) {
            x[0].load(a.init + (size_t)r * d + i);
#pragma unroll
            for (int t = 1; t < SM_; ++t) x[t] = x[0];
        } else {
#pragma unroll
            for (int t = 0; t < SM_; ++t)
                if (t < s) x[t].load_rw(xs + (size_t)t * d + i);
        }
        if (a.has_branch) {
#pragma unroll
            for (int j = 0; j < PA; ++j)
                if (j < a.SA) pa[j].load(a.a + (size_t)j * a.stride_a + (size_t)r * d + i);
#pragma unroll
            for (int j = 0; j < PB; ++j)
                if (j < a.SB) pb[j].load(a.b + (size_t)j * a.stride_b + (size_t)r * d + i);
            if (a.bias) bias.load(a.bias + i);
        }
        // ---- then the arithmetic, element by element of the pack
#pragma unroll
        for (int e = 0; e < E; ++e) {
            float xv[SM_];
#pragma unroll
            for (int t = 0; t < SM_; ++t) xv[t] = t < s ? x[t].v[e] : 0.f;
            if (a.has_branch) {
                float ya = 0.f, yb = 0.f;
#pragma unroll
                for (int j = 0; j < PA; ++j)
                    if (j < a.SA) ya += pa[j].v[e];
                for (int j = PA; j < a.SA; ++j) ya += __ldg(a.a + (size_t)j * a.stride_a + (size_t)r * d + i + e);
                if (a.bias) ya += bias.v[e];
#pragma unroll
                for (int j = 0; j < PB; ++j)
                    if (j < a.SB) yb += pb[j].v[e];
                for (int j = PB; j < a.SB; ++j) yb += __ldg(a.b + (size_t)j * a.stride_b + (size_t)r * d + i + e);
                const float y = a.SB > 0 ? a.scale_a * ya + a.scale_b * yb : a.scale_a * ya;
                float nx[SM_];
#pragma unroll
                for (int t = 0; t < SM_; ++t) {
                    float v = 0.f;
                    if (t < s) {
#pragma unroll
                        for (int f = 0; f < SM_; ++f)
                            if (f < s) v = fmaf(c_mix[f * s + t], xv[f], v);
                        v = fmaf(c_out[t], y, v);
                    }
                    nx[t] = v;
                }
#pragma unroll
                for (int t = 0; t < SM_; ++t) { xv[t] = nx[t]; x[t].v[e] = nx[t]; }
            }
            float u = 0.f;
#pragma unroll
            for (int t = 0; t < SM_; ++t)
                if (t < s) u = fmaf(c_in[t], xv[t], u);
            urow[i + e] = u;
            total += u;
            if (a.read_out) a.read_out[(size_t)m * d + i + e] = u;
        }
        if (a.write_streams) {
#pragma unroll
            for (int t = 0; t < SM_; ++t)
                if (t < s) x[t].store(xs + (size_t)t * d + i);
        }
    }
    if (a.out == nullptr) return;
    T* o = (T*)a.out + (size_t)m * d;
    if (a.gain == nullptr) {
        __syncthreads();
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<T>(urow[i]);
        return;
    }
    float mean = 0.f;
    if (a.center) mean = block_sum(total, scratch) / (float)d;
    float ss = 0.f;
    for (int i = threadIdx.x * E; i < d; i += blockDim.x * E) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float v = urow[i + e] - mean;
            ss += v * v;
        }
    }
    const float var = block_sum(ss, scratch) / (float)d;
    const float rinv = 1.0f / sqrtf(var + a.eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<T>((urow[i] - mean) * rinv * a.gain[i]);
}

template <typename T, int E, int SM_, int PA, int PB>
cudaError_t launch_one(const HyperArgs& h, int M, int threads, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(hyper_fold_norm_kernel<T, E, SM_, PA, PB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return sb::launch(hyper_fold_norm_kernel<T, E, SM_, PA, PB>, dim3(M), dim3(threads), smem, stream, h);
}

template <typename T>
cudaError_t launch_hyper(const HyperArgs& h, int M, size_t smem, cudaStream_t stream) {
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = h.d % 4 == 0 && h.stride_a % 4 == 0 && h.stride_b % 4 == 0 && aligned(h.streams) && aligned(h.init) &&
                     aligned(h.a) && aligned(h.b) && aligned(h.bias);
    auto round32 = [](int n, int most) { n = ((n + 31) / 32) * 32; return n > most ? most : (n < 32 ? 32 : n); };
    // Few rows (a decode step, the head's rows): a thread a column and every partial sum in flight, so that a row
    // is one round of loads.  Many rows: 256 threads; 16-byte packs where there are at most four streams.
    if (M <= 512) return launch_one<T, 1, SMAX, 16, 16>(h, M, round32(h.d, 1024), smem, stream);
    if (vec && h.s <= 4) return launch_one<T, 4, 4, 4, 4>(h, M, round32(h.d / 4, 256), smem, stream);
    return launch_one<T, 1, SMAX, 8, 8>(h, M, round32(h.d, 256), smem, stream);
}

}  // namespace

extern "C" int sb_hyper_fold_norm(float* streams, const float* init, int s, int d, const float* a, int SA,
                                  long long stride_a, float scale_a, const float* b, int SB, long long stride_b,
                                  float scale_b, const float* bias, const float* mix, const float* outw, float mult,
                                  const float* inw, const float* gain, float eps, int center, void* out,
                                  float* read_out, const int* row_index, int M, int out_dtype, cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && d > 0 && s >= 1 && s <= SMAX, "hyper_fold_norm: %d streams of %d (1 to %d streams)", s, d, SMAX);
    SB_REQUIRE(SA >= 0 && SB >= 0 && (SA == 0 || a != nullptr) && (SB == 0 || b != nullptr),
               "hyper_fold_norm: partial sums without a buffer");
    SB_REQUIRE(SB == 0 || SA > 0, "hyper_fold_norm: a second branch without a first");
    if (M == 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    SB_REQUIRE(smem <= 200 * 1024, "hyper_fold_norm: width %d does not fit one block's shared memory", d);
    HyperArgs h;
    h.streams = streams; h.init = init; h.a = a; h.SA = SA; h.stride_a = (size_t)stride_a; h.scale_a = scale_a;
    h.b = b; h.SB = SB; h.stride_b = (size_t)stride_b; h.scale_b = scale_b; h.bias = bias; h.mix = mix;
    h.outw = outw; h.inw = inw; h.gain = gain; h.mult = mult; h.eps = eps; h.center = center; h.out = out;
    h.read_out = read_out; h.row_index = row_index; h.s = s; h.d = d;
    h.has_branch = SA > 0 || bias != nullptr;
    h.write_streams = row_index == nullptr && (h.has_branch || init != nullptr);
    if (out_dtype == SB_F32) launch_hyper<float>(h, M, smem, stream);
    else if (out_dtype == SB_BF16) launch_hyper<__nv_bfloat16>(h, M, smem, stream);
    else SB_REQUIRE(false, "hyper_fold_norm: unknown dtype %d", out_dtype);
    SB_LAUNCH_CHECK();
}
