// Differential attention over paged keys and values, on the CUDA cores.
//
// A query head carries TWO score maps over ONE set of values: its query row is [map 1 | map 2]
// (`dim` dims each), the key row of its KV head likewise, and
//
//   s1_ij = (q1_i . k1_j) * scale ,  s2_ij = (q2_i . k2_j) * scale
//   a1_i = softmax_j(s1_ij) v_j ,    a2_i = softmax_j(s2_ij) v_j        (each map a softmax of its own)
//   o_i  = a1_i - lambda * a2_i
//   out_i = o_i / sqrt(mean_d(o_i^2) + eps) * out_scale                  (per head, over its Dv value dims)
//
// Visible keys: j <= i and (window == 0 or i - j < window or j < keep_first): a sliding window
// that also keeps the first keys of the sequence where they are (distances and rotation unchanged).  The visible keys of a
// query are therefore two runs, [0, min(keep_first, lo)) and [lo, i]; the kernels walk them as one
// run of consecutive indices (`KeyRun`).
//
// Scores, weights, sums, the difference and the norm are float32.  Three kernels:
//   * one block per (token, KV head, key share): decode steps and whatever the tile kernel does not take;
//     with several shares the (max, sum, weighted values) of every map go to scratch and
//   * a merge kernel joins the shares of each map, takes the difference and norms it;
//   * one block per tile of consecutive tokens of a request (prompt portions): a key or value row
//     fetched once serves every query of the tile.
#include <math.h>

#include "common.cuh"

using namespace sb;

namespace {

constexpr int THREADS = 128;
constexpr int KEYS = 128;      // keys per chunk: one per thread
constexpr int SUBS = 8;        // (head, map) rows per pass of the per-token kernel: four heads, so that a group of
                               // four query heads reads its keys and values once
constexpr int DIMMAX = 128;    // dims of one map
constexpr int ROWS = 32;       // (query, head, map) rows of a tile

struct DiffArgs {
    void* out;                 // [N, H*Dv] in T
    const void* q;             // [N, H*2*dim] in T
    const void* k_pool;        // [pages, Hkv, BS, 2*dim] in T
    const void* v_pool;        // [pages, Hkv, BS, Dv] in T
    const int* block_table;
    int table_width;
    const int* token_rows;
    const int* positions;
    int H, Hkv, dim, Dv, BS, window, keep_first;
    float scale, lambda, eps, out_scale;
    int NP;                    // key shares (grid.z)
    float* part_o;             // [N, H*2, NP, Dv]
    float* part_ml;            // [N, H*2, NP, 2]: running maximum and sum
};

// The visible keys of queries at positions first..last as one run of indices 0..total-1.
struct KeyRun {
    int nkeep, lo, total;
    __device__ __forceinline__ KeyRun(int pos_first, int pos_last, int window, int keep_first) {
        lo = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;
        nkeep = min(keep_first, lo);
        total = nkeep + pos_last + 1 - lo;
    }
    __device__ __forceinline__ int key(int v) const { return v < nkeep ? v : lo + (v - nkeep); }
};

__device__ __forceinline__ bool sees(int pos, int key, int window, int keep_first) {
    return key <= pos && (window <= 0 || pos - key < window || key < keep_first);
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 4) diff_attention_kernel(DiffArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    __shared__ __align__(16) float qs[SUBS][DIMMAX];
    __shared__ float w[SUBS][KEYS];
    __shared__ float run_max[SUBS], run_sum[SUBS], rescale[SUBS];
    __shared__ int vrow[KEYS];             // the pool row (page, KV head, slot) of every key of the chunk
    __shared__ float red[33];
    constexpr int VEC = Vec16<T>::N;
    __shared__ __align__(16) float vred[SUBS][THREADS * VEC];      // [row][row group][value dim] of the 16-byte value path
    const int kh = blockIdx.x, n = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.H / a.Hkv, dim = a.dim, Dv = a.Dv, BS = a.BS;
    const int row = a.token_rows[n], pos = a.positions[n];
    const KeyRun run(pos, pos, a.window, a.keep_first);
    // this block's share of the run: equal counts, in order
    const int per = (run.total + a.NP - 1) / a.NP;
    const int lo = (int)blockIdx.z * per;
    const int hi = min(run.total, lo + per);          // exclusive
    const int* table = a.block_table + (size_t)row * a.table_width;
    const T* q = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;
    const bool vec = dim % VEC == 0 && (reinterpret_cast<uintptr_t>(kp) & 15) == 0;
    // Values in 16-byte pieces: LPR neighbouring threads read one value row, the block RP rows at a time, and a
    // thread keeps VEC dims of every row's sum; the row groups are added up (in order) after the last chunk.
    // Taken when a value row is a power of two of such pieces.
    const int LPR = Dv / VEC;
    const bool vvec = Dv % VEC == 0 && LPR <= THREADS && (LPR & (LPR - 1)) == 0 &&
                      (reinterpret_cast<uintptr_t>(vp) & 15) == 0;
    const int RP = vvec ? THREADS / LPR : 1, rg = vvec ? tid / LPR : 0, lp = vvec ? tid % LPR : 0;

    for (int g0 = 0; g0 < G; g0 += SUBS / 2) {
        const int gn = min(SUBS / 2, G - g0), h0 = kh * G + g0, sn = 2 * gn;
        __syncthreads();
        for (int i = tid; i < sn * dim; i += THREADS) {
            const int s = i / dim, d = i - s * dim;          // row s = (head of the pass) * 2 + map
            qs[s][d] = to_float(q[((size_t)n * a.H + h0) * 2 * dim + i]);
        }
        for (int i = sn * dim + tid; i < SUBS * dim; i += THREADS) qs[i / dim][i % dim] = 0.f;
        if (tid < SUBS) { run_max[tid] = -INFINITY; run_sum[tid] = 0.f; rescale[tid] = 0.f; }
        // a row's sums: dims tid and tid + THREADS in [0] and [1], or the VEC dims of the 16-byte value path
        float accv[SUBS][VEC];
#pragma unroll
        for (int s = 0; s < SUBS; ++s)
#pragma unroll
            for (int e = 0; e < VEC; ++e) accv[s][e] = 0.f;
        __syncthreads();
        for (int c0 = lo; c0 < hi; c0 += KEYS) {
            const int nk = min(KEYS, hi - c0);
            if (tid < nk) {
                const int key = run.key(c0 + tid);
                const int page = table[key / BS];
                const int slot = (page * a.Hkv + kh) * BS + key % BS;
                vrow[tid] = slot;
                const T* kr = kp + (size_t)slot * 2 * dim;
                float dot[SUBS];
#pragma unroll
                for (int s = 0; s < SUBS; ++s) dot[s] = 0.f;
                if (vec) {
#pragma unroll 4
                    for (int d = 0; d < dim; d += VEC) {
                        Vec16<T> k1, k2;
                        k1.load(kr + d);
                        k2.load(kr + dim + d);
#pragma unroll
                        for (int e = 0; e < VEC; e += 4) {
                            const float f1[4] = {k1.get(e), k1.get(e + 1), k1.get(e + 2), k1.get(e + 3)};
                            const float f2[4] = {k2.get(e), k2.get(e + 1), k2.get(e + 2), k2.get(e + 3)};
#pragma unroll
                            for (int s = 0; s < SUBS; ++s) {
                                const float4 qv = *reinterpret_cast<const float4*>(&qs[s][d + e]);
                                const float* f = (s & 1) ? f2 : f1;
                                dot[s] = fmaf(qv.x, f[0], dot[s]);
                                dot[s] = fmaf(qv.y, f[1], dot[s]);
                                dot[s] = fmaf(qv.z, f[2], dot[s]);
                                dot[s] = fmaf(qv.w, f[3], dot[s]);
                            }
                        }
                    }
                } else {
                    for (int d = 0; d < dim; ++d) {
                        const float f1 = to_float(kr[d]), f2 = to_float(kr[dim + d]);
#pragma unroll
                        for (int s = 0; s < SUBS; ++s) dot[s] = fmaf(qs[s][d], (s & 1) ? f2 : f1, dot[s]);
                    }
                }
#pragma unroll
                for (int s = 0; s < SUBS; ++s) w[s][tid] = dot[s] * a.scale;
            }
            __syncthreads();
            // running maximum and weights, one warp per row
            for (int s = warp; s < sn; s += THREADS / 32) {
                float mx = -INFINITY;
                for (int t = lane; t < nk; t += 32) mx = fmaxf(mx, w[s][t]);
                mx = warp_max(mx);
                const float m_old = run_max[s], m_new = fmaxf(m_old, mx);
                float sum = 0.f;
                for (int t = lane; t < nk; t += 32) {
                    const float p = expf(w[s][t] - m_new);
                    w[s][t] = p;
                    sum += p;
                }
                sum = warp_sum(sum);
                if (lane == 0) {
                    const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                    rescale[s] = f;
                    run_sum[s] = run_sum[s] * f + sum;
                    run_max[s] = m_new;
                }
            }
            __syncthreads();
            // weighted sum of the values: thread t owns dims t and t + THREADS; both maps read the same values
            if (vvec) {
#pragma unroll
                for (int s = 0; s < SUBS; ++s) {
                    const float f = rescale[s];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) accv[s][e] *= f;
                }
                for (int t0 = 0; t0 < nk; t0 += 4 * RP) {        // four rows' loads in flight per thread
                    Vec16<T> x[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int t = t0 + j * RP + rg;
                        x[j].load(vp + (size_t)vrow[t < nk ? t : 0] * Dv + lp * VEC);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int t = t0 + j * RP + rg;
                        if (t >= nk) continue;
#pragma unroll
                        for (int s = 0; s < SUBS; ++s) {         // rows beyond the pass's heads have weight 0
                            const float ws = w[s][t];
#pragma unroll
                            for (int e = 0; e < VEC; ++e) accv[s][e] = fmaf(ws, x[j].get(e), accv[s][e]);
                        }
                    }
                }
                __syncthreads();
                continue;
            }
#pragma unroll
            for (int s = 0; s < SUBS; ++s) { accv[s][0] *= rescale[s]; accv[s][1] *= rescale[s]; }
#pragma unroll 8
            for (int t = 0; t < nk; ++t) {
                const T* vr = vp + (size_t)vrow[t] * Dv;
                const float v0 = tid < Dv ? to_float(vr[tid]) : 0.f;
                const float v1 = tid + THREADS < Dv ? to_float(vr[tid + THREADS]) : 0.f;
#pragma unroll
                for (int s = 0; s < SUBS; ++s) {
                    if (s >= sn) continue;
                    accv[s][0] = fmaf(w[s][t], v0, accv[s][0]);
                    accv[s][1] = fmaf(w[s][t], v1, accv[s][1]);
                }
            }
            __syncthreads();
        }
        if (vvec) {
            // the row groups' sums, added in the order 0, 1, ...: thread t takes dims t and t + THREADS as below
#pragma unroll
            for (int s = 0; s < SUBS; ++s)
#pragma unroll
                for (int e = 0; e < VEC; e += 4)
                    *reinterpret_cast<float4*>(&vred[s][rg * Dv + lp * VEC + e]) =
                        make_float4(accv[s][e], accv[s][e + 1], accv[s][e + 2], accv[s][e + 3]);
            __syncthreads();
            const int d0 = tid < Dv ? tid : 0, d1 = tid + THREADS < Dv ? tid + THREADS : d0;
#pragma unroll
            for (int s = 0; s < SUBS; ++s) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
                for (int r = 0; r < RP; ++r) {
                    s0 += vred[s][r * Dv + d0];
                    if (Dv > THREADS) s1 += vred[s][r * Dv + d1];
                }
                accv[s][0] = s0;                              // threads beyond Dv hold a copy that nothing reads
                accv[s][1] = s1;
            }
        }
        if (a.NP == 1) {
#pragma unroll
            for (int g = 0; g < SUBS / 2; ++g) {
                if (g >= gn) continue;                       // uniform over the block
                const float f1 = 1.0f / run_sum[2 * g], f2 = a.lambda / run_sum[2 * g + 1];
                const float o0 = tid < Dv ? accv[2 * g][0] * f1 - accv[2 * g + 1][0] * f2 : 0.f;
                const float o1 = tid + THREADS < Dv ? accv[2 * g][1] * f1 - accv[2 * g + 1][1] * f2 : 0.f;
                const float ss = block_sum(o0 * o0 + o1 * o1, red);
                const float r = a.out_scale / sqrtf(ss / (float)Dv + a.eps);
                T* o = (T*)a.out + ((size_t)n * a.H + h0 + g) * Dv;
                if (tid < Dv) o[tid] = from_float<T>(o0 * r);
                if (tid + THREADS < Dv) o[tid + THREADS] = from_float<T>(o1 * r);
            }
        } else {
#pragma unroll
            for (int s = 0; s < SUBS; ++s) {
                if (s >= sn) continue;
                const size_t slot = (((size_t)n * a.H + h0) * 2 + s) * a.NP + blockIdx.z;
                float* o = a.part_o + slot * Dv;
                if (tid < Dv) o[tid] = accv[s][0];
                if (tid + THREADS < Dv) o[tid + THREADS] = accv[s][1];
                if (tid == 0) {                              // an empty share has sum 0 and is skipped by the merge
                    a.part_ml[slot * 2] = run_max[s];
                    a.part_ml[slot * 2 + 1] = run_sum[s];
                }
            }
        }
    }
}

// Joins the key shares of both maps of one (token, head), takes the difference and norms it.
// Shares are added in the order 0, 1, ...; a share without keys (sum 0) is skipped unread.
template <typename T>
__global__ void __launch_bounds__(THREADS) diff_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                                            const float* __restrict__ part_ml, int H, int Dv, int NP,
                                                            float lambda, float eps, float out_scale) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    __shared__ float red[33];
    const int h = blockIdx.x, n = blockIdx.y, tid = threadIdx.x;
    float a[2][2];                           // [map][dims tid, tid + THREADS]
    // Loads go out sixteen shares at a time (both maps' maxima and sums together) and none depends on another's
    // value, so a merge costs a few round trips to L2 however many shares there are.
    constexpr int B = 16;
    const size_t base0 = ((size_t)n * H + h) * 2 * NP;
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + base0;       // [map][share]
    float M[2] = {-INFINITY, -INFINITY};
    for (int p0 = 0; p0 < NP; p0 += B) {
        float2 v[2][B];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int j = 0; j < B; ++j) v[m][j] = p0 + j < NP ? ml[m * NP + p0 + j] : make_float2(0.f, 0.f);
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int j = 0; j < B; ++j)
                if (v[m][j].y > 0.f) M[m] = fmaxf(M[m], v[m][j].x);
    }
    const bool wide = Dv > THREADS;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float L = 0.f, o0 = 0.f, o1 = 0.f;
        for (int p0 = 0; p0 < NP; p0 += B) {
            float2 v[B];
            float x0[B], x1[B];
#pragma unroll
            for (int j = 0; j < B; ++j) v[j] = p0 + j < NP ? ml[m * NP + p0 + j] : make_float2(0.f, 0.f);   // in L1 by now
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const float* po = part_o + (base0 + (size_t)m * NP + p0 + j) * Dv;
                x0[j] = (v[j].y > 0.f && tid < Dv) ? po[tid] : 0.f;                      // an empty share is never read
                x1[j] = (wide && v[j].y > 0.f && tid + THREADS < Dv) ? po[tid + THREADS] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < B; ++j)
                if (v[j].y > 0.f) {
                    const float wgt = expf(v[j].x - M[m]);
                    L += wgt * v[j].y;
                    o0 += wgt * x0[j];
                    o1 += wgt * x1[j];
                }
        }
        a[m][0] = o0 / L;
        a[m][1] = o1 / L;
    }
    const float o0 = tid < Dv ? a[0][0] - lambda * a[1][0] : 0.f;
    const float o1 = tid + THREADS < Dv ? a[0][1] - lambda * a[1][1] : 0.f;
    const float ss = block_sum(o0 * o0 + o1 * o1, red);
    const float r = out_scale / sqrtf(ss / (float)Dv + eps);
    T* o = out + ((size_t)n * H + h) * Dv;
    if (tid < Dv) o[tid] = from_float<T>(o0 * r);
    if (tid + THREADS < Dv) o[tid + THREADS] = from_float<T>(o1 * r);
}

// ----------------------------------------------------------------------------------------
// Prompt portions: a tile of QT consecutive tokens of one request per block and KV head.
// Row r of the tile = ((query * GP + head of the pass) * 2 + map); QT * GP * 2 = ROWS.
//   scores: thread t owns key t of the chunk, keeps ROWS dot products in registers and reads both halves of its
//           key row in 16-byte pieces; rows of map 1 meet the first half, rows of map 2 the second;
//   softmax: a warp per row, running maximum and sum;
//   values: thread t owns value dim t and ROWS partial outputs; weights come from shared memory four keys a load;
//   end: difference of the two maps' rows, the head's RMS over the block's threads, scale.
// dim a multiple of the 16-byte vector, Dv <= 128; other shapes use the kernel above.
struct DiffTileArgs {
    DiffArgs b;
    const int* seq_starts;
    const int* seq_rows;
    const int* seq_first_pos;
    int R, QT, GP;
};

template <typename T>
__global__ void __launch_bounds__(THREADS, 4) diff_attention_tile_kernel(DiffTileArgs ta) {
    sb::pdl_launch_dependents();
    const DiffArgs& a = ta.b;
    extern __shared__ float tsm[];
    const int dim = a.dim, Dv = a.Dv, BS = a.BS, QT = ta.QT, GP = ta.GP;
    float* Qs = tsm;                        // [ROWS][dim]
    float* Ps = Qs + ROWS * dim;            // [ROWS][KEYS]
    __shared__ float run_max[ROWS], run_sum[ROWS], rescale[ROWS];
    __shared__ int vrow[KEYS];
    __shared__ float red[THREADS / 32][ROWS / 2];
    const int kh = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.H / a.Hkv;
    sb::pdl_wait();
    int r = 0, ti = blockIdx.y;
    for (; r < ta.R; ++r) {
        const int nt = (ta.seq_starts[r + 1] - ta.seq_starts[r] + QT - 1) / QT;
        if (ti < nt) break;
        ti -= nt;
    }
    if (r == ta.R) return;
    const int n_first = ta.seq_starts[r] + ti * QT;
    const int nq = min(QT, ta.seq_starts[r + 1] - n_first);
    const int pos_first = ta.seq_first_pos[r] + ti * QT, pos_last = pos_first + nq - 1;
    const KeyRun run(pos_first, pos_last, a.window, a.keep_first);
    const int* table = a.block_table + (size_t)ta.seq_rows[r] * a.table_width;
    const T* q = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;
    constexpr int VEC = Vec16<T>::N;

    for (int g0 = 0; g0 < G; g0 += GP) {
        const int gn = min(GP, G - g0), h0 = kh * G + g0;
        __syncthreads();
        for (int i = tid; i < ROWS * dim; i += THREADS) {
            const int row = i / dim, d = i - row * dim, pr = row >> 1, m = row & 1, qi = pr / GP, g = pr - qi * GP;
            Qs[i] = (qi < nq && g < gn)
                        ? to_float(q[(((size_t)(n_first + qi) * a.H + h0 + g) * 2 + m) * dim + d]) : 0.f;
        }
        if (tid < ROWS) { run_max[tid] = -INFINITY; run_sum[tid] = 0.f; rescale[tid] = 0.f; }
        float acc[ROWS];
#pragma unroll
        for (int row = 0; row < ROWS; ++row) acc[row] = 0.f;
        __syncthreads();
        for (int c0 = 0; c0 < run.total; c0 += KEYS) {
            // ---- scores of this thread's key against all rows
            {
                const bool have = c0 + tid < run.total;
                const int key = have ? run.key(c0 + tid) : 0;
                float dot[ROWS];
#pragma unroll
                for (int row = 0; row < ROWS; ++row) dot[row] = 0.f;
                if (have) {
                    const int page = table[key / BS];
                    const int slot = (page * a.Hkv + kh) * BS + key % BS;
                    vrow[tid] = slot;
                    const T* kr = kp + (size_t)slot * 2 * dim;
                    for (int d = 0; d < dim; d += VEC) {
                        Vec16<T> k1, k2;
                        k1.load(kr + d);
                        k2.load(kr + dim + d);
#pragma unroll
                        for (int e = 0; e < VEC; e += 4) {
                            const float a0 = k1.get(e), a1 = k1.get(e + 1), a2 = k1.get(e + 2), a3 = k1.get(e + 3);
                            const float b0 = k2.get(e), b1 = k2.get(e + 1), b2 = k2.get(e + 2), b3 = k2.get(e + 3);
#pragma unroll
                            for (int row = 0; row < ROWS; ++row) {
                                const float4 qv = *reinterpret_cast<const float4*>(Qs + row * dim + d + e);
                                dot[row] = (row & 1)
                                    ? fmaf(qv.x, b0, fmaf(qv.y, b1, fmaf(qv.z, b2, fmaf(qv.w, b3, dot[row]))))
                                    : fmaf(qv.x, a0, fmaf(qv.y, a1, fmaf(qv.z, a2, fmaf(qv.w, a3, dot[row]))));
                            }
                        }
                    }
                }
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    const int pr = row >> 1, qi = pr / GP, g = pr - qi * GP;
                    const bool ok = have && qi < nq && g < gn && sees(pos_first + qi, key, a.window, a.keep_first);
                    Ps[row * KEYS + tid] = ok ? dot[row] * a.scale : -INFINITY;
                }
            }
            __syncthreads();
            // ---- running maximum and weights, a warp per row
            for (int row = warp; row < ROWS; row += THREADS / 32) {
                float* pr = Ps + row * KEYS;
                float mx = -INFINITY;
                for (int t = lane; t < KEYS; t += 32) mx = fmaxf(mx, pr[t]);
                mx = warp_max(mx);
                const float m_old = run_max[row], m_new = fmaxf(m_old, mx);
                const float base = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
                float sum = 0.f;
                for (int t = lane; t < KEYS; t += 32) {
                    const float p = expf(pr[t] - base);
                    pr[t] = p;
                    sum += p;
                }
                sum = warp_sum(sum);
                if (lane == 0) {
                    const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                    rescale[row] = f;
                    run_sum[row] = run_sum[row] * f + sum;
                    run_max[row] = m_new;
                }
            }
            __syncthreads();
            // ---- weighted values: this thread's value dim, four keys a step
#pragma unroll
            for (int row = 0; row < ROWS; ++row) acc[row] *= rescale[row];
            const int nk = min(KEYS, run.total - c0);
            for (int t = 0; t < nk; t += 4) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    v[j] = (t + j < nk && tid < Dv) ? to_float(vp[(size_t)vrow[t + j] * Dv + tid]) : 0.f;
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    const float4 wv = *reinterpret_cast<const float4*>(Ps + row * KEYS + t);
                    acc[row] = fmaf(wv.x, v[0], fmaf(wv.y, v[1], fmaf(wv.z, v[2], fmaf(wv.w, v[3], acc[row]))));
                }
            }
            __syncthreads();
        }
        // ---- difference of the maps, the head's RMS over the value dims, scale
        float o[ROWS / 2];
#pragma unroll
        for (int pr = 0; pr < ROWS / 2; ++pr) {
            const int qi = pr / GP, g = pr - qi * GP;
            const bool ok = qi < nq && g < gn && tid < Dv;
            o[pr] = ok ? acc[2 * pr] / run_sum[2 * pr] - a.lambda * (acc[2 * pr + 1] / run_sum[2 * pr + 1]) : 0.f;
            const float ss = warp_sum(o[pr] * o[pr]);
            if (lane == 0) red[warp][pr] = ss;
        }
        __syncthreads();
#pragma unroll
        for (int pr = 0; pr < ROWS / 2; ++pr) {
            const int qi = pr / GP, g = pr - qi * GP;
            if (qi >= nq || g >= gn || tid >= Dv) continue;
            float ss = 0.f;
#pragma unroll
            for (int wi = 0; wi < THREADS / 32; ++wi) ss += red[wi][pr];
            const float rr = a.out_scale / sqrtf(ss / (float)Dv + a.eps);
            ((T*)a.out)[((size_t)(n_first + qi) * a.H + h0 + g) * Dv + tid] = from_float<T>(o[pr] * rr);
        }
    }
}

// Two maps' outputs of a head, [a1 | a2] in float32 (the rows a tensor-core kernel left), to the head's output:
// the difference, its RMS over the value dims, the scale.  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(THREADS) diff_combine_kernel(T* __restrict__ out, const float* __restrict__ maps, int rows,
                                                              int Dv, float lambda, float eps, float out_scale) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int r = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    const float* a1 = maps + (size_t)r * 2 * Dv;
    const float* a2 = a1 + Dv;
    float o[8];                                  // Dv <= 256
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        o[j] = d < Dv ? a1[d] - lambda * a2[d] : 0.f;
        ss += o[j] * o[j];
    }
    ss = warp_sum(ss);
    const float rr = out_scale / sqrtf(ss / (float)Dv + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < Dv) out[(size_t)r * Dv + d] = from_float<T>(o[j] * rr);
    }
}

int fill(DiffArgs& a, void* out, const void* q, const void* k_pool, const void* v_pool, const int* block_table,
         int table_width, const int* token_rows, const int* positions, int N, int H, int Hkv, int dim, int Dv,
         int page_size, int window, int keep_first, float scale, float lambda, float eps, float out_scale) {
    SB_REQUIRE(N >= 0 && H > 0 && Hkv > 0 && H % Hkv == 0,
               "attention_diff: %d query heads are no multiple of %d KV heads", H, Hkv);
    SB_REQUIRE(dim >= 1 && dim <= DIMMAX && Dv >= 1 && Dv <= 2 * THREADS,
               "attention_diff: maps of %d dims (at most %d) and values of %d (at most %d)", dim, DIMMAX, Dv, 2 * THREADS);
    SB_REQUIRE(page_size > 0 && table_width > 0, "attention_diff: bad page_size %d or table width %d", page_size,
               table_width);
    SB_REQUIRE(window >= 0 && keep_first >= 0, "attention_diff: window %d or kept keys %d negative", window, keep_first);
    a.out = out; a.q = q; a.k_pool = k_pool; a.v_pool = v_pool; a.block_table = block_table;
    a.table_width = table_width; a.token_rows = token_rows; a.positions = positions; a.H = H; a.Hkv = Hkv;
    a.dim = dim; a.Dv = Dv; a.BS = page_size; a.window = window; a.keep_first = keep_first; a.scale = scale;
    a.lambda = lambda; a.eps = eps; a.out_scale = out_scale; a.NP = 1; a.part_o = nullptr; a.part_ml = nullptr;
    return 0;
}

}  // namespace

extern "C" int sb_attention_diff(void* out, const void* q, const void* k_pool, const void* v_pool,
                                 const int* block_table, int table_width, const int* token_rows,
                                 const int* positions, int N, int H, int Hkv, int dim, int Dv, int page_size,
                                 int window, int keep_first, float scale, float lambda, float eps, float out_scale,
                                 int num_partitions, float* part_o, float* part_ml, int dtype,
                                 cudaStream_t stream) {
    DiffArgs a;
    if (int e = fill(a, out, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, H, Hkv, dim, Dv,
                     page_size, window, keep_first, scale, lambda, eps, out_scale)) return e;
    SB_REQUIRE(N <= 65535, "attention_diff: %d tokens exceed one launch", N);
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 64 &&
                   (num_partitions == 1 || (part_o != nullptr && part_ml != nullptr)),
               "attention_diff: %d key shares (1 to 64; more than one needs scratch buffers)", num_partitions);
    SB_REQUIRE(dtype == SB_F32 || dtype == SB_BF16, "attention_diff: unknown dtype %d", dtype);
    if (N == 0) return 0;
    a.NP = num_partitions; a.part_o = part_o; a.part_ml = part_ml;
    dim3 grid(Hkv, N, num_partitions), mgrid(H, N);
    if (dtype == SB_F32) {
        sb::launch(diff_attention_kernel<float>, grid, dim3(THREADS), 0, stream, a);
        if (num_partitions > 1)
            sb::launch(diff_merge_kernel<float>, mgrid, dim3(THREADS), 0, stream, (float*)out, (const float*)part_o,
                       (const float*)part_ml, H, Dv, num_partitions, lambda, eps, out_scale);
    } else {
        sb::launch(diff_attention_kernel<__nv_bfloat16>, grid, dim3(THREADS), 0, stream, a);
        if (num_partitions > 1)
            sb::launch(diff_merge_kernel<__nv_bfloat16>, mgrid, dim3(THREADS), 0, stream, (__nv_bfloat16*)out,
                       (const float*)part_o, (const float*)part_ml, H, Dv, num_partitions, lambda, eps, out_scale);
    }
    SB_LAUNCH_CHECK();
}

extern "C" int sb_attention_diff_tile_supports(int H, int Hkv, int dim, int Dv, int dtype) {
    const int vec = dtype == SB_BF16 ? 8 : 4;
    return H % Hkv == 0 && dim % vec == 0 && dim >= vec && dim <= DIMMAX && Dv >= 1 && Dv <= THREADS;
}

extern "C" int sb_attention_diff_tile(void* out, const void* q, const void* k_pool, const void* v_pool,
                                      const int* block_table, int table_width, const int* seq_starts,
                                      const int* seq_rows, const int* seq_first_pos, int R, int N, int H, int Hkv,
                                      int dim, int Dv, int page_size, int window, int keep_first, float scale,
                                      float lambda, float eps, float out_scale, int dtype, cudaStream_t stream) {
    SB_REQUIRE(sb_attention_diff_tile_supports(H, Hkv, dim, Dv, dtype),
               "attention_diff_tile: heads %d/%d with maps of %d and values of %d are not served", H, Hkv, dim, Dv);
    SB_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0, "attention_diff_tile: the key pool must be 16-byte aligned");
    SB_REQUIRE(R >= 0, "attention_diff_tile: %d requests", R);
    SB_REQUIRE(dtype == SB_F32 || dtype == SB_BF16, "attention_diff_tile: unknown dtype %d", dtype);
    DiffTileArgs ta;
    if (int e = fill(ta.b, out, q, k_pool, v_pool, block_table, table_width, nullptr, nullptr, N, H, Hkv, dim, Dv,
                     page_size, window, keep_first, scale, lambda, eps, out_scale)) return e;
    if (N == 0 || R == 0) return 0;
    const int G = H / Hkv;
    ta.seq_starts = seq_starts; ta.seq_rows = seq_rows; ta.seq_first_pos = seq_first_pos; ta.R = R;
    ta.GP = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    ta.QT = ROWS / 2 / ta.GP;
    const int tiles = (N + ta.QT - 1) / ta.QT + R;
    SB_REQUIRE(tiles <= 65535, "attention_diff_tile: %d tiles exceed one launch", tiles);
    const size_t smem = (size_t)ROWS * (dim + KEYS) * sizeof(float);
    dim3 grid(Hkv, tiles);
    if (dtype == SB_F32)
        sb::launch(diff_attention_tile_kernel<float>, grid, dim3(THREADS), smem, stream, ta);
    else
        sb::launch(diff_attention_tile_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, ta);
    SB_LAUNCH_CHECK();
}

// maps float32 [N, H, 2, Dv] -> out [N, H, Dv] in the model dtype.
extern "C" int sb_diff_combine(void* out, const float* maps, int N, int H, int Dv, float lambda, float eps,
                               float out_scale, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && H > 0 && Dv >= 1 && Dv <= 256, "diff_combine: bad sizes N=%d H=%d Dv=%d", N, H, Dv);
    SB_REQUIRE(dtype == SB_F32 || dtype == SB_BF16, "diff_combine: unknown dtype %d", dtype);
    if (N == 0) return 0;
    const int rows = N * H, blocks = (rows + THREADS / 32 - 1) / (THREADS / 32);
    if (dtype == SB_F32)
        sb::launch(diff_combine_kernel<float>, dim3(blocks), dim3(THREADS), 0, stream, (float*)out, maps, rows, Dv, lambda,
                   eps, out_scale);
    else
        sb::launch(diff_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(THREADS), 0, stream, (__nv_bfloat16*)out, maps,
                   rows, Dv, lambda, eps, out_scale);
    SB_LAUNCH_CHECK();
}
