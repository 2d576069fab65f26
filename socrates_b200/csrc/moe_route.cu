// Routing of a mixture-of-experts feed-forward, and the small steps around the experts' products.
//
//   logits:      z[n][e] = sum_k x[n][k] * router[e][k]        (float32 weights and sums, a block per token)
//   route:       s = softmax(z) over all E router outputs (float32)
//                c = s + correction                              (the scores experts are CHOSEN by)
//                the E outputs form `groups` equal groups of neighbours; a group's score is its
//                largest c; only the `keep` best groups stay (the others' c count as -inf)
//                the `top` largest c are chosen; their weights are s (no correction, not renormalized)
//                weights[n][e] = s_e for chosen e, else 0 ;  ids[n][k], picked[n][k] = the choices, best first
//   scale:       act[n][e*F + f] *= weights[n][e]                (all experts' activations side by side)
//   passthrough: slab[n][:] = x[n][:] * sum of weights[n][e] over e >= first_identity
//                (router outputs past the real experts stand for "the input itself")
//
// Ties go to the lower index.  One warp routes one token.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

// (value, index) of the largest value over a warp; ties go to the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(
    const float* __restrict__ logits, const float* __restrict__ correction, float* __restrict__ weights,
    int* __restrict__ ids, float* __restrict__ picked, int N, int E, int groups, int keep, int top) {
    sb::pdl_launch_dependents();
    extern __shared__ float rsm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* s = rsm + (size_t)warp * (2 * E + groups);      // scores
    float* c = s + E;                                       // choice scores
    float* gs = c + E;                                      // group scores
    const int n = blockIdx.x * ROUTE_WARPS + warp;
    sb::pdl_wait();
    if (n >= N) return;
    const float* z = logits + (size_t)n * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float p = expf(z[e] - mx);
        s[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        const float p = s[e] * inv;
        s[e] = p;
        c[e] = p + (correction ? correction[e] : 0.f);
        weights[(size_t)n * E + e] = 0.f;
    }
    __syncwarp();
    if (keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
            gs[g] = best;
        }
        __syncwarp();
        // the `keep` best groups are marked with +inf, then every other group's experts are closed
        for (int it = 0; it < keep; ++it) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && (v > bv || bi == 0x7fffffff)) { bv = v; bi = g; }
            }
            warp_argmax(bv, bi);
            if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (!isnan(v) && (v > bv)) { bv = v; bi = e; }
        }
        warp_argmax(bv, bi);
        if (bi == 0x7fffffff) {                 // fewer open experts than `top`: nothing more to choose
            if (lane == 0) { ids[(size_t)n * top + k] = -1; picked[(size_t)n * top + k] = 0.f; }
            continue;
        }
        if (lane == 0) {
            const float p = s[bi];
            weights[(size_t)n * E + bi] = p;
            ids[(size_t)n * top + k] = bi;
            picked[(size_t)n * top + k] = p;
            c[bi] = NAN;                         // taken
        }
        __syncwarp();
    }
}

// A block per (token, four router outputs): the row of x goes to shared memory once (as float32), then each
// warp sums one output over K in a fixed order, whatever the batch holds: lane l takes elements l, l + 32,
// ..., eight loads in flight, four partial sums joined in a fixed tree.
template <typename T>
__global__ void __launch_bounds__(128) moe_logits_kernel(float* __restrict__ logits, const T* __restrict__ x,
                                                         const float* __restrict__ router, int E, int K) {
    sb::pdl_launch_dependents();
    extern __shared__ float xs[];
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * 4 + warp;
    const float* w = router + (size_t)(e < E ? e : 0) * K;
    float wv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = lane + 32 * j < K ? w[lane + 32 * j] : 0.f;     // weights: before the wait
    sb::pdl_wait();
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(x[(size_t)n * K + k]);
    __syncthreads();
    if (e >= E) return;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int k0 = 0; k0 < K; k0 += 256) {
        float nx[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {                       // the next eight are on their way while these are used
            const int k = k0 + 256 + lane + 32 * j;
            nx[j] = k < K ? w[k] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
            const int k = k0 + lane + 32 * j;
            a0 = fmaf(k < K ? xs[k] : 0.f, wv[j], a0);
            a1 = fmaf(k + 32 < K ? xs[k + 32] : 0.f, wv[j + 1], a1);
            a2 = fmaf(k + 64 < K ? xs[k + 64] : 0.f, wv[j + 2], a2);
            a3 = fmaf(k + 96 < K ? xs[k + 96] : 0.f, wv[j + 3], a3);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[j] = nx[j];
    }
    const float total = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) logits[(size_t)n * E + e] = total;
}

template <typename T>
__global__ void __launch_bounds__(256) moe_scale_kernel(T* __restrict__ act, const float* __restrict__ weights,
                                                        int E_total, int experts, int F, size_t total) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const size_t width = (size_t)experts * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width;
        const int e = (int)((i - n * width) / F);
        const float w = weights[n * E_total + e];
        act[i] = from_float<T>(w == 0.f ? 0.f : to_float(act[i]) * w);
    }
}

// F a multiple of the 16-byte vector: a thread scales one vector, whose elements share their expert.
// An expert that was not chosen is not even read: its activations are overwritten with zeros.
template <typename T>
__global__ void __launch_bounds__(256) moe_scale_vec_kernel(T* __restrict__ act, const float* __restrict__ weights,
                                                            int E_total, int experts, int F, size_t total_vec) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const size_t width_vec = (size_t)experts * F / VEC;
    const int f_vec = F / VEC;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width_vec;
        const int e = (int)((i - n * width_vec) / f_vec);
        const float w = weights[n * E_total + e];
        T* p = act + i * VEC;
        if (w == 0.f) {
            *reinterpret_cast<uint4*>(p) = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        Vec16<T> v;
        v.load(p);
        alignas(16) T r[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) r[j] = from_float<T>(v.get(j) * w);
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(r);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_passthrough_kernel(float* __restrict__ slab, const T* __restrict__ x,
                                                              const float* __restrict__ weights, int E_total,
                                                              int first_identity, int d) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int n = blockIdx.x;
    float w = 0.f;
    for (int e = first_identity; e < E_total; ++e) w += weights[(size_t)n * E_total + e];
    for (int i = threadIdx.x; i < d; i += blockDim.x) slab[(size_t)n * d + i] = w * to_float(x[(size_t)n * d + i]);
}

// Routing by a table: token id t uses the experts table[t, 0..top-1] (distinct), each with weight 1 / top.
// Writes the dense weights [N, E] (zero where not chosen) that the scaling kernel reads.  A negative id -1 - j
// stands for feedback[j], a token that an earlier kernel on the stream wrote (as in the embedding).
__global__ void __launch_bounds__(128) moe_table_kernel(float* __restrict__ weights, const int* __restrict__ ids,
                                                        const int* __restrict__ feedback, const int* __restrict__ table,
                                                        int N, int E, int top, int V) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    int id = ids[n];
    if (id < 0 && feedback != nullptr) id = feedback[-1 - id];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const int* row = table + (size_t)id * top;
    const float share = 1.0f / (float)top;
    for (int e = lane; e < E; e += 32) {
        float w = 0.f;
        for (int j = 0; j < top; ++j) w = row[j] == e ? share : w;
        weights[(size_t)n * E + e] = w;
    }
}

}  // namespace

extern "C" int sb_moe_table(float* weights, const int* ids, const int* feedback, const int* table, int N, int E,
                            int top, int V, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && E > 0 && top >= 1 && top <= E && V > 0, "moe_table: bad sizes N=%d E=%d top=%d V=%d", N, E, top, V);
    if (N == 0) return 0;
    sb::launch(moe_table_kernel, dim3((N + 3) / 4), dim3(128), 0, stream, weights, ids, feedback, table, N, E, top, V);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_moe_route(const float* logits, const float* correction, float* weights, int* ids, float* picked,
                            int N, int E, int groups, int keep, int top, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && E > 0 && top >= 1 && top <= E, "moe_route: bad sizes N=%d E=%d top=%d", N, E, top);
    SB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups,
               "moe_route: %d router outputs in %d groups of which %d stay", E, groups, keep);
    SB_REQUIRE(top <= keep * (E / groups), "moe_route: %d choices from %d open experts", top, keep * (E / groups));
    const size_t smem = (size_t)ROUTE_WARPS * (2 * E + groups) * sizeof(float);
    SB_REQUIRE(smem <= 48 * 1024, "moe_route: %d router outputs do not fit a block's shared memory", E);
    if (N == 0) return 0;
    sb::launch(moe_route_kernel, dim3((N + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream,
               logits, correction, weights, ids, picked, N, E, groups, keep, top);
    SB_LAUNCH_CHECK();
}

// logits float32 [N, E] = x [N, K] (model dtype) times router [E, K] (float32), transposed.
extern "C" int sb_moe_logits(float* logits, const void* x, const float* router, int N, int E, int K, int dtype,
                             cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && E > 0 && K > 0, "moe_logits: bad sizes N=%d E=%d K=%d", N, E, K);
    const size_t smem = (size_t)K * sizeof(float);
    SB_REQUIRE(smem <= 160 * 1024, "moe_logits: rows of %d values do not fit a block's shared memory", K);
    SB_REQUIRE((E + 3) / 4 <= 65535 && N <= 2147483647, "moe_logits: too many router outputs");
    if (N == 0) return 0;
    static sb::OncePerDevice once_f, once_b;
    if (dtype == SB_F32) {
        if (smem > 48 * 1024 && !once_f.flag()) {
            cudaFuncSetAttribute(moe_logits_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            once_f.flag() = true;
        }
        sb::launch(moe_logits_kernel<float>, dim3(N, (E + 3) / 4), dim3(128), smem, stream, logits, (const float*)x, router, E, K);
    } else if (dtype == SB_BF16) {
        if (smem > 48 * 1024 && !once_b.flag()) {
            cudaFuncSetAttribute(moe_logits_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            once_b.flag() = true;
        }
        sb::launch(moe_logits_kernel<__nv_bfloat16>, dim3(N, (E + 3) / 4), dim3(128), smem, stream, logits, (const __nv_bfloat16*)x,
                   router, E, K);
    } else {
        SB_REQUIRE(false, "moe_logits: unknown dtype %d", dtype);
    }
    SB_LAUNCH_CHECK();
}

// act [N, experts*F] in the model dtype; weights float32 [N, E_total], the experts' first.
extern "C" int sb_moe_scale(void* act, const float* weights, int N, int E_total, int experts, int F, int dtype,
                            cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && experts > 0 && experts <= E_total && F > 0, "moe_scale: bad sizes N=%d experts=%d/%d F=%d", N,
               experts, E_total, F);
    if (N == 0) return 0;
    const size_t total = (size_t)N * experts * F;
    const int vec = dtype == SB_BF16 ? 8 : 4;
    if (F % vec == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0 && (dtype == SB_F32 || dtype == SB_BF16)) {
        const size_t tv = total / vec;
        const int vblocks = (int)((tv + 255) / 256 < 148 * 16 ? (tv + 255) / 256 : 148 * 16);
        if (dtype == SB_F32)
            sb::launch(moe_scale_vec_kernel<float>, dim3(vblocks), dim3(256), 0, stream, (float*)act, weights, E_total,
                       experts, F, tv);
        else
            sb::launch(moe_scale_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream, (__nv_bfloat16*)act,
                       weights, E_total, experts, F, tv);
        SB_LAUNCH_CHECK();
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    if (dtype == SB_F32)
        sb::launch(moe_scale_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, weights, E_total, experts, F, total);
    else if (dtype == SB_BF16)
        sb::launch(moe_scale_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)act, weights,
                   E_total, experts, F, total);
    else
        SB_REQUIRE(false, "moe_scale: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

// slab float32 [N, d]; x [N, d] in the model dtype.
extern "C" int sb_moe_passthrough(float* slab, const void* x, const float* weights, int N, int E_total,
                                  int first_identity, int d, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && d > 0 && first_identity >= 0 && first_identity <= E_total, "moe_passthrough: bad sizes");
    if (N == 0) return 0;
    if (dtype == SB_F32)
        sb::launch(moe_passthrough_kernel<float>, dim3(N), dim3(256), 0, stream, slab, (const float*)x, weights, E_total,
                   first_identity, d);
    else if (dtype == SB_BF16)
        sb::launch(moe_passthrough_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, slab, (const __nv_bfloat16*)x,
                   weights, E_total, first_identity, d);
    else
        SB_REQUIRE(false, "moe_passthrough: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}
