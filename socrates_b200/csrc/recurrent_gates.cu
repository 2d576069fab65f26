// Two gated recurrences whose gates read only the current token, so that a prompt portion is one
// walk over its tokens with the state in registers.
//
// min_gru: one state value per channel.
//     z = sigmoid(pz + bz) ,  u = px + bx ,  c = u + 1/2 (u >= 0)  |  sigmoid(u) (u < 0)
//     S <- (1 - z) S + z c ;  y = S * silu(pg)
//   pz, px, pg are columns [0, W), [W, 2W), [2W, 3W) of one matrix product.
//
// gated_linear_attention: a matrix state per head in which the forget gate also decides what is written.
//     q = silu(pq) ,  f = l + (1 - l) sigmoid(pf + bf)      (per head and key channel; l the lower bound)
//     S <- diag(f) S + (1 - f) v^T ;  o = S^T q
//     y = o / sqrt(mean(o^2) + eps) * w                     (per head, over its value dims)
//
// States are float32 and live in the request's state slot; gates, decays, the recurrences and the
// norm are float32; only the products arrive in the model dtype and y leaves in it.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------ min_gru
struct MinGruArgs {
    const void* proj;          // [N, stride] in T
    long long stride;
    const float* bz;           // [W] or null
    const float* bx;           // [W] or null
    float* state;              // [rows, W]
    void* out;                 // [N, W] in T
    const int* seq_starts;
    const int* seq_rows;
    int W;
};

// The recurrence S <- a S + b (a = 1 - z, b = z c) is linear in S, so a request's tokens are cut into
// `segs` segments that run side by side: every thread (a channel, a segment) first walks its segment from a
// zero state and keeps the product of its a's; the segments' results are joined in order through shared memory
// (the state at a segment's start = what the earlier segments leave); then it walks its segment again from its
// true start state and writes the outputs.  One segment (a decode step): a single walk.
template <typename T>
__device__ __forceinline__ void gru_inputs(const T* row, int W, float bz, float bx, float& z, float& c, float& gate) {
    z = sigmoidf_(to_float(row[0]) + bz);
    const float u = to_float(row[W]) + bx;
    c = u >= 0.f ? u + 0.5f : sigmoidf_(u);
    const float gz = to_float(row[2 * W]);
    gate = gz * sigmoidf_(gz);
}

template <typename T>
__global__ void __launch_bounds__(1024) min_gru_kernel(MinGruArgs a, int segs) {
    sb::pdl_launch_dependents();
    extern __shared__ float carry[];            // [segs][32] products of a, then [segs][32] states from zero
    const int lane = threadIdx.x, sg = threadIdx.y;
    const int c = blockIdx.x * 32 + lane, r = blockIdx.y, W = a.W;
    const bool live = c < W;
    const float bz = (live && a.bz) ? a.bz[c] : 0.f, bx = (live && a.bx) ? a.bx[c] : 0.f;
    sb::pdl_wait();
    const int t0 = a.seq_starts[r], t1 = a.seq_starts[r + 1];
    if (t0 >= t1) return;
    const int per = (t1 - t0 + segs - 1) / segs;
    const int lo = min(t1, t0 + sg * per), hi = min(t1, lo + per);
    float* sp = a.state + (size_t)a.seq_rows[r] * W + c;
    const T* p = (const T*)a.proj + c;
    T* y = (T*)a.out + c;
    constexpr int U = 4;                        // tokens whose loads and gates are made before the chain runs over them
    float S = (segs == 1 && live) ? *sp : 0.f;
    if (segs > 1) {
        float A = 1.f;
        if (live) {
            for (int tc = lo; tc < hi; tc += U) {
                float z[U], cand[U], gate[U];
#pragma unroll
                for (int j = 0; j < U; ++j) gru_inputs(p + (size_t)min(tc + j, hi - 1) * a.stride, W, bz, bx, z[j], cand[j], gate[j]);
#pragma unroll
                for (int j = 0; j < U; ++j)
                    if (tc + j < hi) { S = fmaf(z[j], cand[j] - S, S); A *= 1.f - z[j]; }
            }
        }
        carry[sg * 32 + lane] = A;
        carry[(segs + sg) * 32 + lane] = S;
        __syncthreads();
        S = live ? *sp : 0.f;                   // the request's state, carried through the segments before this one
        for (int k = 0; k < sg; ++k) S = fmaf(carry[k * 32 + lane], S, carry[(segs + k) * 32 + lane]);
        if (sg == segs - 1 && live)             // the last segment also knows the state the request leaves
            *sp = fmaf(carry[sg * 32 + lane], S, carry[(segs + sg) * 32 + lane]);
    }
    if (!live) return;
    for (int tc = lo; tc < hi; tc += U) {
        float z[U], cand[U], gate[U];
#pragma unroll
        for (int j = 0; j < U; ++j) gru_inputs(p + (size_t)min(tc + j, hi - 1) * a.stride, W, bz, bx, z[j], cand[j], gate[j]);
#pragma unroll
        for (int j = 0; j < U; ++j) {
            if (tc + j < hi) {
                S = fmaf(z[j], cand[j] - S, S);            // (1 - z) S + z c
                y[(size_t)(tc + j) * W] = from_float<T>(S * gate[j]);
            }
        }
    }
    if (segs == 1) *sp = S;
}

// ------------------------------------------------------------------------------------ gated linear attention
struct GlaArgs {
    const void* proj;          // [N, stride] in T: q at q_off (H*D), f at f_off (H*D), v at v_off (H*Dv)
    long long stride;
    int q_off, f_off, v_off;
    const float* f_bias;       // [H*D] or null
    const float* lower;        // [H*D] or null (0)
    const float* norm_w;       // [Dv]
    float* state;              // [rows, H, D, Dv]
    void* out;                 // [N, H*Dv] in T
    float* raw_o;              // [N, H*Dv]
    const int* seq_starts;
    const int* seq_rows;
    int H, D, Dv;
    float eps;
    // Long portions are cut into `segs` segments that run side by side (the recurrence is linear in S with a
    // diagonal decay): mode 1 walks every segment from a zero state and leaves its end state and the product of
    // its forget gates in `seg_scratch`; mode 2 joins what the earlier segments left, in order, walks again
    // and writes the outputs.  Mode 0: one segment, one walk.
    int mode, segs;
    float* seg_scratch;        // [R, segs + 1, H, D, Dv + 1]: per segment the end state and (last column) the gate product; slot `segs`: the state at the start
};

constexpr int RG = 16;         // threads that share a column of the state
constexpr int COLS = 8;        // columns of a block
constexpr int TB = 16;         // tokens staged at a time
constexpr int GTHREADS = RG * COLS;

// The walk over a request's tokens is serial, so nothing in it may wait for memory: while the threads walk
// the 16 tokens of one chunk, the raw gate and query values of the NEXT chunk are already on their way into
// registers; gates, lower bound and SiLU are applied when they are moved to shared memory.
template <typename T, int DR>
__global__ void __launch_bounds__(GTHREADS) gla_kernel(GlaArgs a) {
    sb::pdl_launch_dependents();
    constexpr int DP = RG * DR;                       // padded key dims
    constexpr int NE = TB * DP / GTHREADS;            // (token, key dim) pairs a thread stages per chunk
    __shared__ float fs[TB][DP + 4], qs[TB][DP + 4], vs[TB][COLS], os[TB][COLS];
    __shared__ float low_s[DP], fb_s[DP];
    const int h = blockIdx.x, r = blockIdx.y / a.segs, seg = blockIdx.y - r * a.segs, c0 = blockIdx.z * COLS;
    const int tid = threadIdx.x, rg = tid & (RG - 1), cj = tid / RG, j = c0 + cj;
    const int D = a.D, Dv = a.Dv, H = a.H;
    for (int d = tid; d < DP; d += GTHREADS) {        // constants of the model: before the wait
        low_s[d] = (d < D && a.lower) ? a.lower[h * D + d] : 0.f;
        fb_s[d] = (d < D && a.f_bias) ? a.f_bias[h * D + d] : 0.f;
    }
    sb::pdl_wait();
    const int r0 = a.seq_starts[r], r1 = a.seq_starts[r + 1];
    if (r0 >= r1) return;
    const int per = (r1 - r0 + a.segs - 1) / a.segs;
    const int t0 = min(r1, r0 + seg * per), t1 = min(r1, t0 + per);      // this block's tokens
    const T* proj = (const T*)a.proj;
    const bool col = j < Dv;
    float* sp = a.state + ((size_t)a.seq_rows[r] * H + h) * D * Dv + j;
    const size_t SW = (size_t)Dv + 1;                                    // a scratch row: Dv state values, then the gate product
    float* seg_base = a.seg_scratch + ((size_t)r * (a.segs + 1) * H + h) * D * SW;
    const size_t seg_stride = (size_t)H * D * SW;
    float S[DR], A[DR];
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = rg + RG * ii;                   // thread rg owns rows rg, rg + 16, ...
        const bool live = col && i < D;
        A[ii] = 1.f;
        S[ii] = 0.f;
        if (a.mode == 0) {
            S[ii] = live ? sp[(size_t)i * Dv] : 0.f;
        } else if (a.mode == 1) {
            if (seg == 0 && live) seg_base[a.segs * seg_stride + (size_t)i * SW + j] = sp[(size_t)i * Dv];     // kept for mode 2
        } else if (live) {
            float v = seg_base[a.segs * seg_stride + (size_t)i * SW + j];
            for (int k = 0; k < seg; ++k) {
                const float* sk = seg_base + k * seg_stride + (size_t)i * SW;
                v = fmaf(sk[Dv], v, sk[j]);
            }
            S[ii] = v;
        }
    }
    float rf[NE], rq[NE], rv;
    auto fetch = [&](int tc) {
#pragma unroll
        for (int k = 0; k < NE; ++k) {
            const int i = tid + k * GTHREADS, tt = i / DP, d = i - tt * DP;
            rf[k] = rq[k] = 0.f;
            if (d < D && tc + tt < t1) {
                const T* row = proj + (size_t)(tc + tt) * a.stride + h * D + d;
                rf[k] = to_float(row[a.f_off]);
                rq[k] = to_float(row[a.q_off]);
            }
        }
        const int tt = tid / COLS, c = tid - tt * COLS;            // TB * COLS = GTHREADS: one value a thread
        rv = (c0 + c < Dv && tc + tt < t1) ? to_float(proj[(size_t)(tc + tt) * a.stride + a.v_off + h * Dv + c0 + c]) : 0.f;
    };
    fetch(t0);
    for (int tc = t0; tc < t1; tc += TB) {
        const int nt = min(TB, t1 - tc);
        __syncthreads();                              // the walk over the chunk before is over
#pragma unroll
        for (int k = 0; k < NE; ++k) {
            const int i = tid + k * GTHREADS, tt = i / DP, d = i - tt * DP;
            const float l = low_s[d];
            fs[tt][d] = d < D ? l + (1.0f - l) * sigmoidf_(rf[k] + fb_s[d]) : 1.f;      // rows past D keep a zero state
            qs[tt][d] = rq[k] * sigmoidf_(rq[k]);
        }
        vs[tid / COLS][tid % COLS] = rv;
        __syncthreads();
        if (tc + TB < t1) fetch(tc + TB);             // in flight while the chunk is walked
        // the state of one token feeds the next through one multiply-add only; the dot products and their shuffles
        // of four tokens run side by side (the chunk's tail past nt holds f = 1, v = q = 0 from an earlier chunk
        // or garbage that is never written out, and the state is walked over real tokens only)
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt][cj];
            float o = 0.f;
#pragma unroll
            for (int ii = 0; ii < DR; ++ii) {
                const float f = fs[tt][rg + RG * ii];
                S[ii] = fmaf(f, S[ii] - v, v);        // f S + (1 - f) v
                A[ii] *= f;
                o = fmaf(S[ii], qs[tt][rg + RG * ii], o);
            }
            if (a.mode == 1) continue;                // only the end state and the gate product are wanted
#pragma unroll
            for (int sh = 1; sh < RG; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
            if (rg == 0) os[tt][cj] = o;
        }
        __syncthreads();
        if (a.mode != 1) {
            const int tt = tid / COLS, c = tid - tt * COLS;
            if (tt < nt && c0 + c < Dv) a.raw_o[(size_t)(tc + tt) * H * Dv + h * Dv + c0 + c] = os[tt][c];
        }
    }
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = rg + RG * ii;
        if (!(col && i < D)) continue;
        if (a.mode == 1) {
            float* sk = seg_base + seg * seg_stride + (size_t)i * SW;
            sk[j] = S[ii];
            if (j == 0) sk[Dv] = A[ii];               // the same in every column; column 0 writes it
        } else if (seg == a.segs - 1) {
            sp[(size_t)i * Dv] = S[ii];               // the last segment leaves the request's state
        }
    }
}

// y = o / sqrt(mean(o^2) + eps) * w, a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) gla_out_kernel(GlaArgs a, int N) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= N * a.H) return;
    const int Dv = a.Dv;
    const float* o = a.raw_o + (size_t)item * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    const float rinv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
    T* y = (T*)a.out + (size_t)item * Dv;
    for (int j = lane; j < Dv; j += 32) y[j] = from_float<T>(o[j] * rinv * a.norm_w[j]);
}

template <typename T>
int launch_gla(GlaArgs a, int R, int N, cudaStream_t stream) {
    const dim3 grid(a.H, R * a.segs, (a.Dv + COLS - 1) / COLS);
    for (int mode = a.segs > 1 ? 1 : 0; mode <= (a.segs > 1 ? 2 : 0); ++mode) {
        a.mode = mode;
        if (a.D <= RG * 4) sb::launch(gla_kernel<T, 4>, grid, dim3(GTHREADS), 0, stream, a);
        else if (a.D <= RG * 8) sb::launch(gla_kernel<T, 8>, grid, dim3(GTHREADS), 0, stream, a);
        else sb::launch(gla_kernel<T, 16>, grid, dim3(GTHREADS), 0, stream, a);
    }
    sb::launch(gla_out_kernel<T>, dim3((N * a.H + 3) / 4), dim3(128), 0, stream, a, N);
    SB_LAUNCH_CHECK();
}

}  // namespace

// `longest`: an upper bound of the tokens any request brings (the launch shape depends on it, not the result).
extern "C" int sb_min_gru(void* out, const void* proj, long long stride, const float* bz, const float* bx,
                          float* state, const int* seq_starts, const int* seq_rows, int R, int W, int longest,
                          int dtype, cudaStream_t stream) {
    SB_REQUIRE(R >= 0 && W > 0 && stride >= 3LL * W, "min_gru: %d channels in rows of %lld", W, stride);
    SB_REQUIRE(R <= 65535, "min_gru: %d requests exceed one launch", R);
    if (R == 0) return 0;
    MinGruArgs a;
    a.proj = proj; a.stride = stride; a.bz = bz; a.bx = bx; a.state = state; a.out = out;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.W = W;
    int segs = (longest + 15) / 16;             // at least 16 tokens a segment, at most 32 segments
    segs = segs < 1 ? 1 : (segs > 32 ? 32 : segs);
    const dim3 grid((W + 31) / 32, R), block(32, segs);
    const size_t smem = (size_t)2 * segs * 32 * sizeof(float);
    if (dtype == SB_F32) sb::launch(min_gru_kernel<float>, grid, block, smem, stream, a, segs);
    else if (dtype == SB_BF16) sb::launch(min_gru_kernel<__nv_bfloat16>, grid, block, smem, stream, a, segs);
    else SB_REQUIRE(false, "min_gru: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

extern "C" int sb_gated_linear_attention_supports(int D, int Dv) { return D >= 1 && D <= 256 && Dv >= 1; }

// Segments a request's tokens are cut into when the longest request brings at most `longest` tokens: at least
// 128 tokens a segment, at most 16 segments.
extern "C" int sb_gated_linear_attention_segments(int longest) {
    const int s = (longest + 127) / 128;
    return s < 1 ? 1 : (s > 16 ? 16 : s);
}

extern "C" int sb_gated_linear_attention(void* out, const void* proj, long long stride, int q_off, int f_off,
                                         int v_off, const float* f_bias, const float* lower, const float* norm_w,
                                         float* state, const int* seq_starts, const int* seq_rows, int R, int H,
                                         int D, int Dv, float eps, int dtype, float* raw_o, int N, int segs,
                                         float* seg_scratch, cudaStream_t stream) {
    SB_REQUIRE(segs >= 1 && segs <= 16 && (segs == 1 || seg_scratch != nullptr),
               "gated_linear_attention: %d segments (1 to 16; more than one needs scratch)", segs);
    SB_REQUIRE(R >= 0 && H > 0 && sb_gated_linear_attention_supports(D, Dv),
               "gated_linear_attention: %d heads of %d (keys, at most 256) and %d (values) dims", H, D, Dv);
    SB_REQUIRE(R * segs <= 65535 && (Dv + COLS - 1) / COLS <= 65535, "gated_linear_attention: %d requests exceed one launch", R);
    SB_REQUIRE(raw_o != nullptr && N >= 0, "gated_linear_attention: scratch for %d tokens is missing", N);
    if (R == 0 || N == 0) return 0;
    GlaArgs a;
    a.proj = proj; a.stride = stride; a.q_off = q_off; a.f_off = f_off; a.v_off = v_off; a.f_bias = f_bias;
    a.lower = lower; a.norm_w = norm_w; a.state = state; a.out = out; a.raw_o = raw_o;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.H = H; a.D = D; a.Dv = Dv; a.eps = eps;
    a.mode = 0; a.segs = segs; a.seg_scratch = seg_scratch;
    if (dtype == SB_F32) return launch_gla<float>(a, R, N, stream);
    if (dtype == SB_BF16) return launch_gla<__nv_bfloat16>(a, R, N, stream);
    SB_REQUIRE(false, "gated_linear_attention: unknown dtype %d", dtype);
}
