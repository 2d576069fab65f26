// Paged causal softmax attention whose scores are mixed across the heads before the softmax
// ("talking heads"), on the CUDA cores, with a sigmoid gate on the output.
//
//   r_g(i, j) = q_g(i) . k_kv(g)(j)                      raw score of head g (grouped keys: kv(g) = g / (H / Hkv))
//   s_h(i, j) = scale * sum_g talk[h][g] r_g(i, j)        every head's score reads every head's raw score
//   keys j <= i (and i - j < window, if one is given)
//   o_h(i) = softmax_j(s_h(i, j)) v_kv(h)(j) * sigmoid(gate_h(i))      (gate per head and value dim, optional)
//
// Because a head's score needs all heads' raw scores, a block serves ALL heads of a tile of consecutive
// tokens of one request: rows = (query, head), ordered by KV head so that the rows that share a key or
// value row are neighbours.  Per chunk of 128 keys:
//   raw scores: thread t owns key t; for each KV head it reads its key row in 16-byte pieces and forms the
//               dot products of that head's rows four at a time (q comes from shared memory);
//   mixing:     thread t mixes the raw scores of its key, query by query, masks and scales;
//   softmax:    a warp per row, running maximum and sum;
//   values:     thread t owns value dim t; it reads sixteen value rows of a KV head and adds them into that
//               head's rows, whose sums sit in shared memory (rows are too many for registers).
// Scores, weights and sums are float32.  A decode step gives every token a tile of its own (one query)
// and cuts its keys into shares, merged by the kernel of attention_reduce.cuh.
#include <math.h>

#include "common.cuh"
#include "attention_reduce.cuh"

using namespace sb;

namespace {

constexpr int THREADS = 256;    // two threads a key (and a value dim): each takes every other group of rows
constexpr int KEYS = 128;
constexpr int RGRP = 4;        // rows whose dot products a thread forms side by side
constexpr int VG = 16;         // value rows a thread holds at a time

struct TalkArgs {
    void* out;                 // [N, H*Dv] in T
    const void* q;             // [N, H*Dk] in T
    const void* k_pool;        // [pages, Hkv, BS, Dk] in T
    const void* v_pool;        // [pages, Hkv, BS, Dv] in T
    const int* block_table;
    int table_width;
    const int* seq_starts;
    const int* seq_rows;
    const int* seq_first_pos;
    int R;
    const float* talk;         // [H, H]: (to, from)
    const void* gate;          // [N, gate_stride] in T, column h * Dv + d; or null
    long long gate_stride;
    int H, Hkv, Dk, Dv, BS, window;
    float scale;
    int QT;                    // queries of a tile
    int NP;                    // key shares (grid.y); > 1: results go to part_o / part_ml
    float* part_o;             // [N, H, NP, Dv]
    float* part_ml;            // [N, H, NP, 2]
};

template <typename T>
__global__ void __launch_bounds__(THREADS) talk_attention_kernel(TalkArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ __align__(16) float sm[];
    const int H = a.H, Hkv = a.Hkv, G = H / Hkv, Dk = a.Dk, Dv = a.Dv, BS = a.BS, QT = a.QT;
    const int RK = QT * G, ROWS = QT * H;              // rows of one KV head; all rows
    const int DkP = (Dk + 3) & ~3;                     // q rows padded to 16 bytes
    float* Qs = sm;                                    // [ROWS][DkP]
    float* Praw = Qs + (size_t)ROWS * DkP;             // [ROWS][KEYS]
    float* Pmix = Praw + (size_t)ROWS * KEYS;          // [ROWS][KEYS]
    float* Acc = Pmix + (size_t)ROWS * KEYS;           // [ROWS][Dv]
    float* talk_s = Acc + (size_t)ROWS * Dv;           // [H][H]
    float* run_max = talk_s + H * H;                   // [ROWS] each
    float* run_sum = run_max + ROWS;
    float* rescale = run_sum + ROWS;
    int* pg = reinterpret_cast<int*>(rescale + ROWS);  // [KEYS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kt = tid & (KEYS - 1), part = tid / KEYS;     // the key (value dim) of this thread, and which half of the rows
    for (int i = tid; i < H * H; i += THREADS) talk_s[i] = a.talk[i];     // weights: before the wait
    sb::pdl_wait();
    // tiles are served last first: a request's late tiles see the most keys and should not start last
    int r = 0, ti = (int)(gridDim.x - 1 - blockIdx.x);
    for (; r < a.R; ++r) {
        const int nt = (a.seq_starts[r + 1] - a.seq_starts[r] + QT - 1) / QT;
        if (ti < nt) break;
        ti -= nt;
    }
    if (r == a.R) return;
    const int n_first = a.seq_starts[r] + ti * QT;
    const int nq = min(QT, a.seq_starts[r + 1] - n_first);
    const int pos_first = a.seq_first_pos[r] + ti * QT, pos_last = pos_first + nq - 1;
    const int lo_tile = (a.window > 0 && pos_first + 1 > a.window) ? pos_first + 1 - a.window : 0;
    const int per = (pos_last + 1 - lo_tile + a.NP - 1) / a.NP;
    const int lo = lo_tile + (int)blockIdx.y * per;
    const int hi = min(pos_last + 1, lo + per);        // exclusive
    const int* table = a.block_table + (size_t)a.seq_rows[r] * a.table_width;
    const T* q = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;
    constexpr int VEC = Vec16<T>::N;
    const bool vec_keys = Dk % VEC == 0 && (reinterpret_cast<uintptr_t>(kp) & 15) == 0;

    // row (kh, qi, g) = kh * RK + qi * G + g holds query qi of head kh * G + g
    for (int i = tid; i < ROWS * DkP; i += THREADS) {
        const int row = i / DkP, d = i - row * DkP;
        const int kh = row / RK, rr = row - kh * RK, qi = rr / G, g = rr - qi * G;
        Qs[i] = (qi < nq && d < Dk) ? to_float(q[((size_t)(n_first + qi) * H + kh * G + g) * Dk + d]) : 0.f;
    }
    for (int i = tid; i < ROWS * Dv; i += THREADS) Acc[i] = 0.f;
    for (int i = tid; i < ROWS; i += THREADS) { run_max[i] = -INFINITY; run_sum[i] = 0.f; rescale[i] = 0.f; }
    __syncthreads();

    for (int c0 = lo; c0 < hi; c0 += KEYS) {
        const int nk = min(KEYS, hi - c0);
        const int key = c0 + kt;
        const bool have = kt < nk;
        // ---- raw scores of this thread's key against every row
        int page = 0;
        if (have) { page = table[key / BS]; pg[kt] = page; }
        // (KV head, group of four rows) pairs are dealt to the two threads of a key in turn
        const int groups = (RK + RGRP - 1) / RGRP;
        for (int unit = part; unit < Hkv * groups; unit += THREADS / KEYS) {
            const int kh = unit / groups, r0 = (unit - kh * groups) * RGRP;
            const T* kr = kp + (((size_t)page * Hkv + kh) * BS + key % BS) * Dk;
            {
                const int rn = min(RGRP, RK - r0);
                const float* qrow = Qs + (size_t)(kh * RK + r0) * DkP;
                float dot[RGRP];
#pragma unroll
                for (int j = 0; j < RGRP; ++j) dot[j] = 0.f;
                if (have) {
                    if (vec_keys) {
                        // four 16-byte pieces at a time, the next four on their way while these are used
                        Vec16<T> kv[4], nx[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (u * VEC < Dk) kv[u].load(kr + u * VEC);
                        for (int d0 = 0; d0 < Dk; d0 += 4 * VEC) {
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (d0 + (4 + u) * VEC < Dk) nx[u].load(kr + d0 + (4 + u) * VEC);
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int d = d0 + u * VEC;
                                if (d >= Dk) break;
#pragma unroll
                                for (int e = 0; e < VEC; e += 4) {
                                    const float k0 = kv[u].get(e), k1 = kv[u].get(e + 1), k2 = kv[u].get(e + 2), k3 = kv[u].get(e + 3);
#pragma unroll
                                    for (int j = 0; j < RGRP; ++j) {
                                        if (j < rn) {
                                            const float4 qv = *reinterpret_cast<const float4*>(qrow + j * DkP + d + e);
                                            dot[j] = fmaf(qv.x, k0, fmaf(qv.y, k1, fmaf(qv.z, k2, fmaf(qv.w, k3, dot[j]))));
                                        }
                                    }
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) kv[u] = nx[u];
                        }
                    } else {
                        for (int d = 0; d < Dk; ++d) {
                            const float kf = to_float(kr[d]);
#pragma unroll
                            for (int j = 0; j < RGRP; ++j)
                                if (j < rn) dot[j] = fmaf(qrow[j * DkP + d], kf, dot[j]);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < RGRP; ++j)
                    if (j < rn) Praw[(size_t)(kh * RK + r0 + j) * KEYS + kt] = dot[j];
            }
        }
        __syncthreads();
        // ---- every head's score from all heads' raw scores of the same (query, key); mask; scale
        for (int unit = part; unit < QT * H; unit += THREADS / KEYS) {
            const int qi = unit / H, h = unit - qi * H;
            const int pos = pos_first + qi;
            const int lo_q = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
            const bool seen = have && qi < nq && key <= pos && key >= lo_q;
            {
                float s = -INFINITY;
                if (seen) {
                    s = 0.f;
                    const float* tw = talk_s + h * H;
                    for (int kh = 0; kh < Hkv; ++kh)
                        for (int g = 0; g < G; ++g)
                            s = fmaf(tw[kh * G + g], Praw[(size_t)(kh * RK + qi * G + g) * KEYS + kt], s);
                    s *= a.scale;
                }
                Pmix[(size_t)((h / G) * RK + qi * G + h % G) * KEYS + kt] = s;
            }
        }
        __syncthreads();
        // ---- running maximum and weights, a warp per row
        for (int row = warp; row < ROWS; row += THREADS / 32) {
            float* pr = Pmix + (size_t)row * KEYS;
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
        // ---- weighted values: this thread's value dim; sixteen value rows of a KV head at a time
        for (int d0 = 0; d0 < Dv; d0 += KEYS) {
            const int dim = d0 + kt;
            if (dim >= Dv) continue;
            // the two threads of a value dim share the KV heads when their number is even (each reads its own value
            // rows), else the rows of every KV head
            const bool by_head = Hkv % 2 == 0;
            for (int kh = by_head ? part : 0; kh < Hkv; kh += by_head ? 2 : 1) {
                // sixteen value rows at a time, the next sixteen on their way while these are added
                float v[VG], vn[VG];
                auto fetch = [&](float* dst, int t0) {
#pragma unroll
                    for (int j = 0; j < VG; ++j) {
                        const int t = t0 + j;
                        dst[j] = t < nk ? to_float(vp[(((size_t)pg[t] * Hkv + kh) * BS + (c0 + t) % BS) * Dv + dim]) : 0.f;
                    }
                };
                fetch(v, 0);
                for (int t0 = 0; t0 < nk; t0 += VG) {
                    if (t0 + VG < nk) fetch(vn, t0 + VG);
                    for (int rr = by_head ? 0 : part; rr < RK; rr += by_head ? 1 : 2) {
                        const int row = kh * RK + rr;
                        float acc = Acc[(size_t)row * Dv + dim];
                        if (t0 == 0) acc *= rescale[row];
                        const float* w = Pmix + (size_t)row * KEYS + t0;
#pragma unroll
                        for (int j = 0; j < VG; j += 4) {
                            const float4 wv = *reinterpret_cast<const float4*>(w + j);
                            acc = fmaf(wv.x, v[j], fmaf(wv.y, v[j + 1], fmaf(wv.z, v[j + 2], fmaf(wv.w, v[j + 3], acc))));
                        }
                        Acc[(size_t)row * Dv + dim] = acc;
                    }
#pragma unroll
                    for (int j = 0; j < VG; ++j) v[j] = vn[j];
                }
            }
        }
        __syncthreads();
    }
    // ---- results
    for (int row = 0; row < ROWS; ++row) {
        const int kh = row / RK, rr = row - kh * RK, qi = rr / G, g = rr - qi * G;
        if (qi >= nq) continue;
        const int h = kh * G + g, n = n_first + qi;
        for (int dim = tid; dim < Dv; dim += THREADS) {
            float f = 1.0f;
            if (a.gate) {
                const float z = to_float(((const T*)a.gate)[(size_t)n * a.gate_stride + (size_t)h * Dv + dim]);
                f = 1.0f / (1.0f + expf(-z));
            }
            const float o = Acc[(size_t)row * Dv + dim] * f;
            if (a.NP == 1) {
                ((T*)a.out)[((size_t)n * H + h) * Dv + dim] = from_float<T>(o / run_sum[row]);
            } else {
                a.part_o[(((size_t)n * H + h) * a.NP + blockIdx.y) * Dv + dim] = o;
            }
        }
        if (a.NP > 1 && tid == 0) {
            const size_t slot = ((size_t)n * H + h) * a.NP + blockIdx.y;
            a.part_ml[slot * 2] = run_max[row];
            a.part_ml[slot * 2 + 1] = run_sum[row];
        }
    }
}

// ----------------------------------------------------------------------------------------
// The same attention for ONE long prompt portion in the bfloat16 engine, with both products on the tensor
// cores through the engine's matrix product: the portion's keys are gathered out of their pages into one
// matrix per KV head (values transposed, twice side by side), the raw scores of a block of queries are one
// product per KV head (float32 sums over the bfloat16 q and k), a kernel mixes them across the heads in place,
// another masks, takes the softmax in float32 and writes every weight as two bfloat16 terms [high | low], and the weighted
// values are one more product per KV head over both terms.  The kernels here are the three steps between
// the products.
struct TalkDenseArgs {
    const __nv_bfloat16* q;        // [N, H*Dk]
    const __nv_bfloat16* k_pool;   // [pages, Hkv, BS, Dk]
    const __nv_bfloat16* v_pool;   // [pages, Hkv, BS, Dv]
    const int* table;              // the request's row of the block table
    __nv_bfloat16* Kc;             // [Hkv, Cp, Dk]
    __nv_bfloat16* Vt;             // [Hkv, Dv, 2*Cp]
    __nv_bfloat16* Qg;             // [Hkv, G*nb, Dk]
    const float* S;                // [Hkv, G*nb, Cp] raw scores
    __nv_bfloat16* P;              // [Hkv, G*nb, 2*Cp] weights, high and low terms
    const float* O;                // [Hkv, G*nb, Dv]
    __nv_bfloat16* out;            // [N, H*Dv]
    const __nv_bfloat16* gate;     // [N, gate_stride] or null
    long long gate_stride;
    const float* talk;             // [H, H]
    int H, Hkv, Dk, Dv, BS, C, Cp, n0, nb, pos0, window;     // C keys; queries n0 .. n0+nb-1 at positions pos0 ..
    float scale;
};

// keys of 64 positions of one KV head: rows into Kc, value rows transposed into both halves of Vt
__global__ void __launch_bounds__(256) talk_gather_kv_kernel(TalkDenseArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ __nv_bfloat16 vt[];       // [64][Dv + 2]
    const int j0 = blockIdx.x * 64, kh = blockIdx.y, Dk = a.Dk, Dv = a.Dv, P2 = Dv + 2;
    sb::pdl_wait();
    for (int i = threadIdx.x; i < 64 * Dk; i += blockDim.x) {
        const int jj = i / Dk, d = i - jj * Dk, j = j0 + jj;
        __nv_bfloat16 v = __float2bfloat16_rn(0.f);
        if (j < a.C) v = a.k_pool[(((size_t)a.table[j / a.BS] * a.Hkv + kh) * a.BS + j % a.BS) * Dk + d];
        a.Kc[((size_t)kh * a.Cp + j) * Dk + d] = v;
    }
    for (int i = threadIdx.x; i < 64 * Dv; i += blockDim.x) {
        const int jj = i / Dv, e = i - jj * Dv, j = j0 + jj;
        __nv_bfloat16 v = __float2bfloat16_rn(0.f);
        if (j < a.C) v = a.v_pool[(((size_t)a.table[j / a.BS] * a.Hkv + kh) * a.BS + j % a.BS) * Dv + e];
        vt[jj * P2 + e] = v;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * Dv; i += blockDim.x) {
        const int e = i / 64, jj = i - e * 64;
        const __nv_bfloat16 v = vt[jj * P2 + e];
        __nv_bfloat16* row = a.Vt + ((size_t)kh * Dv + e) * 2 * a.Cp;
        row[j0 + jj] = v;
        row[a.Cp + j0 + jj] = v;
    }
}

// queries of the block, the heads of a KV head one under the other
__global__ void __launch_bounds__(256) talk_gather_q_kernel(TalkDenseArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int i = blockIdx.x, G = a.H / a.Hkv;
    for (int c = threadIdx.x; c < a.H * a.Dk; c += blockDim.x) {
        const int h = c / a.Dk, d = c - h * a.Dk, kh = h / G, g = h - kh * G;
        a.Qg[((size_t)kh * G * a.nb + (size_t)g * a.nb + i) * a.Dk + d] = a.q[(size_t)(a.n0 + i) * a.H * a.Dk + c];
    }
}

// every head's scaled score from all heads' raw scores of the same (query, key), IN PLACE: a thread owns one
// (query, key), reads its HB raw scores once and writes the mixed ones over them
template <int HB>
__global__ void __launch_bounds__(256) talk_mix_kernel(TalkDenseArgs a, float* S) {
    sb::pdl_launch_dependents();
    __shared__ float tw[HB * HB];
    const int i = blockIdx.x, H = a.H, G = H / a.Hkv, Cp = a.Cp;
    for (int c = threadIdx.x; c < HB * HB; c += blockDim.x) {
        const int h = c / HB, g = c - h * HB;
        tw[c] = (h < H && g < H) ? a.talk[h * H + g] * a.scale : 0.f;
    }
    sb::pdl_wait();
    __syncthreads();
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= Cp || j > a.pos0 + i) return;              // keys behind the query are never read
    float raw[HB];
#pragma unroll
    for (int g = 0; g < HB; ++g) {
        const int kh = g / G, gg = g - kh * G;
        raw[g] = g < H ? S[((size_t)kh * G * a.nb + (size_t)gg * a.nb + i) * Cp + j] : 0.f;
    }
    for (int h = 0; h < H; ++h) {
        float m = 0.f;
#pragma unroll
        for (int g = 0; g < HB; ++g) m = fmaf(tw[h * HB + g], raw[g], m);
        const int kh = h / G, gg = h - kh * G;
        S[((size_t)kh * G * a.nb + (size_t)gg * a.nb + i) * Cp + j] = m;
    }
}

// one (query, head): mask the mixed scores, softmax, two bfloat16 terms a weight
__global__ void __launch_bounds__(256) talk_mix_softmax_kernel(TalkDenseArgs a) {
    sb::pdl_launch_dependents();
    extern __shared__ float row[];              // Cp mixed scores
    __shared__ float scratch[33];
    const int i = blockIdx.x, h = blockIdx.y, H = a.H, G = H / a.Hkv, Cp = a.Cp;
    sb::pdl_wait();
    const int pos = a.pos0 + i;
    const int lo = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
    const int hi = min(pos, a.C - 1);           // keys lo .. hi are seen
    float mx = -INFINITY;
    const float* mixed = a.S + ((size_t)(h / G) * G * a.nb + (size_t)(h % G) * a.nb + i) * Cp;
    for (int j = lo + threadIdx.x; j <= hi; j += blockDim.x) {
        const float s = mixed[j];
        row[j] = s;
        mx = fmaxf(mx, s);
    }
    // block maximum (block_sum's scratch, the same order every time)
    mx = warp_max(mx);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, scratch[w]);
    float sum = 0.f;
    for (int j = lo + threadIdx.x; j <= hi; j += blockDim.x) {
        const float p = expf(row[j] - mx);
        row[j] = p;
        sum += p;
    }
    const float inv = 1.0f / block_sum(sum, scratch);
    const int kh = h / G, gg = h - kh * G;
    (void)H;
    __nv_bfloat16* pr = a.P + ((size_t)kh * G * a.nb + (size_t)gg * a.nb + i) * 2 * Cp;
    for (int j = threadIdx.x; j < Cp; j += blockDim.x) {
        float p = (j >= lo && j <= hi) ? row[j] * inv : 0.f;
        const __nv_bfloat16 ph = __float2bfloat16_rn(p);
        pr[j] = ph;
        pr[Cp + j] = __float2bfloat16_rn(p - __bfloat162float(ph));
    }
}

// the heads' outputs back in their places, gated
__global__ void __launch_bounds__(256) talk_finish_kernel(TalkDenseArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    const int i = blockIdx.x, G = a.H / a.Hkv, n = a.n0 + i;
    for (int c = threadIdx.x; c < a.H * a.Dv; c += blockDim.x) {
        const int h = c / a.Dv, e = c - h * a.Dv, kh = h / G, g = h - kh * G;
        float o = a.O[((size_t)kh * G * a.nb + (size_t)g * a.nb + i) * a.Dv + e];
        if (a.gate) {
            const float z = __bfloat162float(a.gate[(size_t)n * a.gate_stride + c]);
            o *= 1.0f / (1.0f + expf(-z));
        }
        a.out[(size_t)n * a.H * a.Dv + c] = __float2bfloat16_rn(o);
    }
}

size_t talk_smem(int QT, int H, int Dk, int Dv) {
    const size_t rows = (size_t)QT * H, dkp = (Dk + 3) & ~3;
    return (rows * (dkp + 2 * KEYS + Dv + 3) + (size_t)H * H + KEYS) * sizeof(float);
}

int gcd_(int a, int b) { return b == 0 ? a : gcd_(b, a % b); }

}  // namespace

// Queries of a tile for prompt portions: a multiple of the smallest count that makes the rows of a KV head a
// multiple of four (the dot products are formed four rows at a time); one query when even that does not fit.
// 0: the shape is not served.
extern "C" int sb_attention_talk_tile(int H, int Hkv, int Dk, int Dv) {
    if (H < 1 || Hkv < 1 || H % Hkv || Dk < 1 || Dv < 1) return 0;
    const int G = H / Hkv, unit = RGRP / gcd_(G, RGRP);
    // few heads: about 48 rows and 100 KB, two blocks an SM; many heads: up to 96 rows and 200 KB in one block, so
    // that several queries still share every key and value row
    const int rows = H <= 24 ? 48 : 96;
    const size_t room = H <= 24 ? 100 * 1024 : 200 * 1024;
    int QT = unit * (rows / (H * unit) > 0 ? rows / (H * unit) : 1);
    while (QT > unit && talk_smem(QT, H, Dk, Dv) > room) QT -= unit;
    if (talk_smem(QT, H, Dk, Dv) > room) QT = 1;
    return talk_smem(QT, H, Dk, Dv) <= 220 * 1024 ? QT : 0;
}

extern "C" int sb_attention_talk(void* out, const void* q, const void* k_pool, const void* v_pool,
                                 const int* block_table, int table_width, const int* seq_starts, const int* seq_rows,
                                 const int* seq_first_pos, int R, const float* talk, const void* gate,
                                 long long gate_stride, int N, int H, int Hkv, int Dk, int Dv, int page_size,
                                 int window, float scale, int queries_per_tile, int num_partitions, float* part_o,
                                 float* part_ml, int dtype, cudaStream_t stream) {
    SB_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0, "attention_talk: %d query heads are no multiple of %d KV heads", H, Hkv);
    SB_REQUIRE(talk != nullptr, "attention_talk: the mixing matrix is missing");
    SB_REQUIRE(page_size > 0 && table_width > 0 && window >= 0 && R >= 0 && N >= 0, "attention_talk: bad sizes");
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 64 &&
                   (num_partitions == 1 || (part_o != nullptr && part_ml != nullptr)),
               "attention_talk: %d key shares (1 to 64; more than one needs scratch buffers)", num_partitions);
    const int QT = queries_per_tile > 0 ? queries_per_tile : sb_attention_talk_tile(H, Hkv, Dk, Dv);
    SB_REQUIRE(QT > 0 && talk_smem(QT, H, Dk, Dv) <= 220 * 1024,
               "attention_talk: %d heads of %d (keys) and %d (values) dims do not fit a block's shared memory", H, Dk, Dv);
    if (N == 0 || R == 0) return 0;
    TalkArgs a;
    a.out = out; a.q = q; a.k_pool = k_pool; a.v_pool = v_pool; a.block_table = block_table; a.table_width = table_width;
    a.seq_starts = seq_starts; a.seq_rows = seq_rows; a.seq_first_pos = seq_first_pos; a.R = R; a.talk = talk;
    a.gate = gate; a.gate_stride = gate_stride; a.H = H; a.Hkv = Hkv; a.Dk = Dk; a.Dv = Dv; a.BS = page_size;
    a.window = window; a.scale = scale; a.QT = QT; a.NP = num_partitions; a.part_o = part_o; a.part_ml = part_ml;
    const int tiles = (N + QT - 1) / QT + R;
    const size_t smem = talk_smem(QT, H, Dk, Dv);
    const dim3 grid(tiles, num_partitions), rgrid(H, N);
    SB_REQUIRE(N <= 65535, "attention_talk: %d tokens exceed one launch", N);
    static sb::OncePerDevice once_f, once_b;
    if (dtype == SB_F32) {
        if (!once_f.flag()) {
            cudaFuncSetAttribute(talk_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            once_f.flag() = true;
        }
        sb::launch(talk_attention_kernel<float>, grid, dim3(THREADS), smem, stream, a);
        if (num_partitions > 1)
            sb::launch(attn_reduce_kernel<float>, rgrid, dim3(128), 0, stream, (float*)out, (const float*)part_o,
                       (const float*)part_ml, H, Dv, num_partitions);
    } else if (dtype == SB_BF16) {
        if (!once_b.flag()) {
            cudaFuncSetAttribute(talk_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            once_b.flag() = true;
        }
        sb::launch(talk_attention_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, a);
        if (num_partitions > 1)
            sb::launch(attn_reduce_kernel<__nv_bfloat16>, rgrid, dim3(128), 0, stream, (__nv_bfloat16*)out,
                       (const float*)part_o, (const float*)part_ml, H, Dv, num_partitions);
    } else {
        SB_REQUIRE(false, "attention_talk: unknown dtype %d", dtype);
    }
    SB_LAUNCH_CHECK();
}

// Steps of the tensor-core form for one long prompt portion (see TalkDenseArgs).  step 0: gather keys and values of
// the request's C keys; 1: gather the block's queries; 2: mix, mask and softmax the block's raw scores; 3: write
// the block's outputs.  All matrices are the caller's; Cp = C rounded up to a multiple of 64.
extern "C" int sb_attention_talk_dense(int step, const void* q, const void* k_pool, const void* v_pool, const int* table,
                                       void* Kc, void* Vt, void* Qg, const float* S, void* P, const float* O, void* out,
                                       const void* gate, long long gate_stride, const float* talk, int H, int Hkv, int Dk,
                                       int Dv, int page_size, int C, int Cp, int n0, int nb, int pos0, int window,
                                       float scale, cudaStream_t stream) {
    SB_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0 && H <= 64, "attention_talk_dense: %d heads over %d KV heads (at most 64)", H, Hkv);
    SB_REQUIRE(C > 0 && Cp >= C && Cp % 64 == 0 && nb > 0 && step >= 0 && step <= 3, "attention_talk_dense: bad sizes");
    SB_REQUIRE(nb <= 65535 && Cp / 64 <= 65535, "attention_talk_dense: a block of %d queries over %d keys exceeds one launch", nb, Cp);
    TalkDenseArgs a;
    a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
    a.table = table; a.Kc = (__nv_bfloat16*)Kc; a.Vt = (__nv_bfloat16*)Vt; a.Qg = (__nv_bfloat16*)Qg; a.S = S;
    a.P = (__nv_bfloat16*)P; a.O = O; a.out = (__nv_bfloat16*)out; a.gate = (const __nv_bfloat16*)gate;
    a.gate_stride = gate_stride; a.talk = talk; a.H = H; a.Hkv = Hkv; a.Dk = Dk; a.Dv = Dv; a.BS = page_size; a.C = C;
    a.Cp = Cp; a.n0 = n0; a.nb = nb; a.pos0 = pos0; a.window = window; a.scale = scale;
    if (step == 0) {
        const size_t smem = (size_t)64 * (Dv + 2) * sizeof(__nv_bfloat16);
        SB_REQUIRE(smem <= 48 * 1024, "attention_talk_dense: value heads of %d dims", Dv);
        sb::launch(talk_gather_kv_kernel, dim3(Cp / 64, Hkv), dim3(256), smem, stream, a);
    } else if (step == 1) {
        sb::launch(talk_gather_q_kernel, dim3(nb), dim3(256), 0, stream, a);
    } else if (step == 2) {
        const size_t smem = (size_t)Cp * sizeof(float);
        SB_REQUIRE(smem <= 200 * 1024, "attention_talk_dense: %d keys do not fit a block's shared memory", Cp);
        static sb::OncePerDevice once;
        if (!once.flag()) {
            cudaFuncSetAttribute(talk_mix_softmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            once.flag() = true;
        }
        float* mixed = const_cast<float*>(S);
        const dim3 mgrid(nb, (Cp + 255) / 256);
        if (H <= 8) sb::launch(talk_mix_kernel<8>, mgrid, dim3(256), 0, stream, a, mixed);
        else if (H <= 16) sb::launch(talk_mix_kernel<16>, mgrid, dim3(256), 0, stream, a, mixed);
        else if (H <= 32) sb::launch(talk_mix_kernel<32>, mgrid, dim3(256), 0, stream, a, mixed);
        else sb::launch(talk_mix_kernel<64>, mgrid, dim3(256), 0, stream, a, mixed);
        sb::launch(talk_mix_softmax_kernel, dim3(nb, H), dim3(256), smem, stream, a);
    } else {
        sb::launch(talk_finish_kernel, dim3(nb), dim3(256), 0, stream, a);
    }
    SB_LAUNCH_CHECK();
}
