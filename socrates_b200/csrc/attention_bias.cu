// Paged causal attention with capped scores, a bias by distance and a gate per head, on the
// CUDA cores.  Every token of the step is a query of its own (prompt portions and decoded
// tokens alike); the step's keys and values are already in the pages.
//
//   s_ij = (q_i . k_j) * scale
//   s_ij = cap * tanh(s_ij / cap)                  (cap > 0)
//   s_ij += dist_bias[h][min(i - j, L - 1)]        (a table by distance, made on the host)
//   keys j with 0 <= i - j < window                (window 0: all keys)
//   o_i = softmax_j(s_ij) v_j * sigmoid(gate_i[h]) (gate optional; one per head, or one per head and value dim)
//   with a sink: p_ij = exp(s_ij) / (exp(sink) + sum_j exp(s_ij)), one more term in the denominator that has no value
//
// Keys have `Dk` dims and values `Dv`; they may differ, and the two pools are shaped accordingly.
// Scores, softmax weights and the weighted sum are float32.  One block serves the query heads of
// one KV head for one token, running over the visible keys in chunks with a running maximum.
#include <math.h>

#include "common.cuh"
#include "attention_reduce.cuh"

using namespace sb;

namespace {

constexpr int THREADS = 128;
constexpr int KEYS = 128;      // keys per chunk: one per thread
constexpr int HEADS = 4;       // query heads per pass over the keys
constexpr int DMAX = 576;

struct BiasAttnArgs {
    void* out;                 // [N, Hq*Dv] in T
    const void* q;             // [N, Hq*Dk] in T
    const void* k_pool;        // [pages, Hkv, BS, Dk] in T
    const void* v_pool;        // [pages, Hkv, BS, Dv] in T
    const int* block_table;
    int table_width;
    const int* token_rows;
    const int* positions;
    const void* gate;          // [N, gate_stride] in T, head h at column h; or null
    long long gate_stride;
    const float* dist_bias;    // [Hq, L] or null
    int L;
    int Hq, Hkv, Dk, Dv, BS, window;
    float scale, cap;
    int NP;                    // key partitions (grid.z); > 1: results go to part_o / part_ml and are merged after
    float* part_o;             // [N, Hq, NP, Dv]
    float* part_ml;            // [N, Hq, NP, 2]: running maximum and sum
    int gate_per_dim;          // 0: gate column h; 1: gate column h * Dv + value dim
    int has_sink;              // the softmax denominator holds exp(sink) beside the keys' terms
    float sink;
};

// The sigmoid gate of output (token n, head h, value dim d); 1 without a gate.
template <typename T>
__device__ __forceinline__ float gate_factor(const BiasAttnArgs& a, int n, int h, int d) {
    if (a.gate == nullptr) return 1.0f;
    const size_t col = a.gate_per_dim ? (size_t)h * a.Dv + d : (size_t)h;
    const float z = to_float(((const T*)a.gate)[(size_t)n * a.gate_stride + col]);
    return 1.0f / (1.0f + expf(-z));
}

template <typename T>
__global__ void __launch_bounds__(THREADS) bias_attention_kernel(BiasAttnArgs a) {
    sb::pdl_launch_dependents();
    sb::pdl_wait();
    __shared__ float qs[HEADS][DMAX];
    __shared__ float w[HEADS][KEYS];
    __shared__ float run_max[HEADS], run_sum[HEADS], rescale[HEADS];
    __shared__ int pg[KEYS];               // the page of every key of the chunk
    const int kh = blockIdx.x, n = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.Hq / a.Hkv, Dk = a.Dk, Dv = a.Dv, BS = a.BS;
    const int row = a.token_rows[n], pos = a.positions[n];
    const int lo_all = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
    // this block's share of the visible keys lo_all..pos: equal counts, in order
    const int per = (pos + 1 - lo_all + a.NP - 1) / a.NP;
    const int lo = lo_all + (int)blockIdx.z * per;
    const int hi = min(pos + 1, lo + per);          // exclusive
    const int* table = a.block_table + (size_t)row * a.table_width;
    const T* q = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;

    for (int g0 = 0; g0 < G; g0 += HEADS) {
        const int gn = min(HEADS, G - g0), h0 = kh * G + g0;
        __syncthreads();
        for (int i = tid; i < gn * Dk; i += THREADS) {
            const int g = i / Dk, d = i - g * Dk;
            qs[g][d] = to_float(q[((size_t)n * a.Hq + h0 + g) * Dk + d]);
        }
        // the sink is a key without a value: the first share of the keys starts from its term
        const bool sink_here = a.has_sink && blockIdx.z == 0;
        if (tid < HEADS) { run_max[tid] = sink_here ? a.sink : -INFINITY; run_sum[tid] = sink_here ? 1.f : 0.f; rescale[tid] = 0.f; }
        float acc[HEADS][2];
#pragma unroll
        for (int g = 0; g < HEADS; ++g) acc[g][0] = acc[g][1] = 0.f;
        __syncthreads();
        for (int c0 = lo; c0 < hi; c0 += KEYS) {
            const int nk = min(KEYS, hi - c0);
            // scores of one key per thread, for all heads of the pass
            if (tid < nk) {
                const int key = c0 + tid;
                const int page = table[key / BS];
                pg[tid] = page;
                const T* kr = kp + (((size_t)page * a.Hkv + kh) * BS + key % BS) * Dk;
                float dot[HEADS];
#pragma unroll
                for (int g = 0; g < HEADS; ++g) dot[g] = 0.f;
                constexpr int VEC = Vec16<T>::N;
                if (Dk % VEC == 0 && (reinterpret_cast<uintptr_t>(kp) & 15) == 0) {
#pragma unroll 4
                    for (int d = 0; d < Dk; d += VEC) {         // 16-byte loads, several in flight
                        Vec16<T> kv;
                        kv.load(kr + d);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            const float kf = kv.get(e);
#pragma unroll
                            for (int g = 0; g < HEADS; ++g) dot[g] = fmaf(qs[g][d + e], kf, dot[g]);
                        }
                    }
                } else {
                    for (int d = 0; d < Dk; ++d) {
                        const float kf = to_float(kr[d]);
#pragma unroll
                        for (int g = 0; g < HEADS; ++g) dot[g] = fmaf(qs[g][d], kf, dot[g]);
                    }
                }
                const int dist = min(pos - key, a.L - 1);
#pragma unroll
                for (int g = 0; g < HEADS; ++g) {
                    if (g >= gn) continue;
                    float s = dot[g] * a.scale;
                    if (a.cap > 0.f) s = a.cap * tanhf(s / a.cap);
                    if (a.dist_bias) s += a.dist_bias[(size_t)(h0 + g) * a.L + dist];
                    w[g][tid] = s;
                }
            }
            __syncthreads();
            // running maximum and weights, one warp per head
            for (int g = warp; g < gn; g += THREADS / 32) {
                float mx = -INFINITY;
                for (int t = lane; t < nk; t += 32) mx = fmaxf(mx, w[g][t]);
                mx = warp_max(mx);
                const float m_old = run_max[g], m_new = fmaxf(m_old, mx);
                float sum = 0.f;
                for (int t = lane; t < nk; t += 32) {
                    const float p = expf(w[g][t] - m_new);
                    w[g][t] = p;
                    sum += p;
                }
                sum = warp_sum(sum);
                if (lane == 0) {
                    const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                    rescale[g] = f;
                    run_sum[g] = run_sum[g] * f + sum;
                    run_max[g] = m_new;
                }
            }
            __syncthreads();
            // weighted sum of the values: thread t owns dims t and t + THREADS
#pragma unroll
            for (int g = 0; g < HEADS; ++g) { acc[g][0] *= rescale[g]; acc[g][1] *= rescale[g]; }
#pragma unroll 8
            for (int t = 0; t < nk; ++t) {                      // the addresses come from shared memory: loads overlap
                const int key = c0 + t;
                const T* vr = vp + (((size_t)pg[t] * a.Hkv + kh) * BS + key % BS) * Dv;
                const float v0 = tid < Dv ? to_float(vr[tid]) : 0.f;
                const float v1 = tid + THREADS < Dv ? to_float(vr[tid + THREADS]) : 0.f;
#pragma unroll
                for (int g = 0; g < HEADS; ++g) {
                    if (g >= gn) continue;
                    acc[g][0] = fmaf(w[g][t], v0, acc[g][0]);
                    acc[g][1] = fmaf(w[g][t], v1, acc[g][1]);
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int g = 0; g < HEADS; ++g) {
            if (g >= gn) continue;
            const int h = h0 + g;
            // the gate scales the output, so it may scale every part
            const float f0 = tid < Dv ? gate_factor<T>(a, n, h, tid) : 1.0f;
            const float f1 = tid + THREADS < Dv ? gate_factor<T>(a, n, h, tid + THREADS) : 1.0f;
            if (a.NP == 1) {
                const float f = 1.0f / run_sum[g];
                T* o = (T*)a.out + ((size_t)n * a.Hq + h) * Dv;
                if (tid < Dv) o[tid] = from_float<T>(acc[g][0] * f * f0);
                if (tid + THREADS < Dv) o[tid + THREADS] = from_float<T>(acc[g][1] * f * f1);
            } else {
                const size_t slot = ((size_t)n * a.Hq + h) * a.NP + blockIdx.z;
                float* o = a.part_o + slot * Dv;
                if (tid < Dv) o[tid] = acc[g][0] * f0;
                if (tid + THREADS < Dv) o[tid + THREADS] = acc[g][1] * f1;
                if (tid == 0) {                          // an empty part has sum 0 and is skipped by the merge
                    a.part_ml[slot * 2] = run_max[g];
                    a.part_ml[slot * 2 + 1] = run_sum[g];
                }
            }
        }
    }
}


// ----------------------------------------------------------------------------------------
// The same attention for prompt portions, a tile of consecutive tokens of one request per block.
// A tile's queries see almost the same keys, so a key or value row fetched once serves all of them:
// 32 rows (queries x the query heads of a pass) share every 128-key chunk.
//   scores: thread t owns key t of the chunk, keeps 32 dot products in registers and reads its key row
//           in 16-byte pieces; q comes from shared memory four dims a load;
//   softmax: a warp per row, running maximum and sum as in the kernel above;
//   values: thread t owns value dim t and 32 partial outputs; weights come from shared memory four keys a load.
// Scores, weights and sums are float32.  Dv <= 128 and 16-byte key rows; other shapes use the kernel above.
constexpr int ROWS = 32;       // 64 rows need 255 registers a thread (two blocks of four warps an SM); 32 leave room for four (measured: 1.21 ms a launch against 1.38 with three and 1.50 with 64 rows)

struct TileArgs {
    BiasAttnArgs b;
    const int* seq_starts;
    const int* seq_rows;
    const int* seq_first_pos;
    int R, QT, GP;             // requests; queries per tile and heads per pass (QT * GP = ROWS)
};

template <typename T>
__global__ void __launch_bounds__(THREADS, 4) bias_attention_tile_kernel(TileArgs ta) {
    sb::pdl_launch_dependents();
    const BiasAttnArgs& a = ta.b;
    extern __shared__ float tsm[];
    const int Dk = a.Dk, Dv = a.Dv, BS = a.BS, QT = ta.QT, GP = ta.GP;
    float* Qs = tsm;                        // [ROWS][Dk]
    float* Ps = Qs + ROWS * Dk;             // [ROWS][KEYS]
    __shared__ float run_max[ROWS], run_sum[ROWS], rescale[ROWS];
    __shared__ int pg[KEYS];
    const int kh = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.Hq / a.Hkv;
    sb::pdl_wait();
    // which request and which of its tiles
    int r = 0, ti = blockIdx.y;
    for (; r < ta.R; ++r) {
        const int nt = (ta.seq_starts[r + 1] - ta.seq_starts[r] + QT - 1) / QT;
        if (ti < nt) break;
        ti -= nt;
    }
    if (r == ta.R) return;
    const int n_first = ta.seq_starts[r] + ti * QT;
    const int nq = min(QT, ta.seq_starts[r + 1] - n_first);                 // queries in this tile
    const int pos_first = ta.seq_first_pos[r] + ti * QT, pos_last = pos_first + nq - 1;
    const int lo_tile = (a.window > 0 && pos_first + 1 > a.window) ? pos_first + 1 - a.window : 0;
    const int* table = a.block_table + (size_t)ta.seq_rows[r] * a.table_width;
    const T* q = (const T*)a.q;
    const T* kp = (const T*)a.k_pool;
    const T* vp = (const T*)a.v_pool;
    constexpr int VEC = Vec16<T>::N;

    for (int g0 = 0; g0 < G; g0 += GP) {
        const int gn = min(GP, G - g0), h0 = kh * G + g0;
        __syncthreads();
        // row = query * GP + head of the pass; rows past the tile's queries or the pass's heads stay zero
        for (int i = tid; i < ROWS * Dk; i += THREADS) {
            const int row = i / Dk, d = i - row * Dk, qi = row / GP, g = row - qi * GP;
            Qs[i] = (qi < nq && g < gn) ? to_float(q[((size_t)(n_first + qi) * a.Hq + h0 + g) * Dk + d]) : 0.f;
        }
        if (tid < ROWS) { run_max[tid] = a.has_sink ? a.sink : -INFINITY; run_sum[tid] = a.has_sink ? 1.f : 0.f; rescale[tid] = 0.f; }
        float acc[ROWS];
#pragma unroll
        for (int row = 0; row < ROWS; ++row) acc[row] = 0.f;
        __syncthreads();
        for (int c0 = lo_tile; c0 <= pos_last; c0 += KEYS) {
            // ---- scores of this thread's key against all rows
            {
                const int key = c0 + tid;
                const bool have = key <= pos_last;
                float dot[ROWS];
#pragma unroll
                for (int row = 0; row < ROWS; ++row) dot[row] = 0.f;
                if (have) {
                    const int page = table[key / BS];
                    pg[tid] = page;
                    const T* kr = kp + (((size_t)page * a.Hkv + kh) * BS + key % BS) * Dk;
                    for (int d = 0; d < Dk; d += VEC) {
                        Vec16<T> kv;
                        kv.load(kr + d);
#pragma unroll
                        for (int e = 0; e < VEC; e += 4) {
                            const float k0 = kv.get(e), k1 = kv.get(e + 1), k2 = kv.get(e + 2), k3 = kv.get(e + 3);
#pragma unroll
                            for (int row = 0; row < ROWS; ++row) {
                                const float4 qv = *reinterpret_cast<const float4*>(Qs + row * Dk + d + e);
                                dot[row] = fmaf(qv.x, k0, fmaf(qv.y, k1, fmaf(qv.z, k2, fmaf(qv.w, k3, dot[row]))));
                            }
                        }
                    }
                }
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    const int qi = row / GP, g = row - qi * GP;
                    const int pos = pos_first + qi;
                    const int lo = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
                    float sc = -INFINITY;
                    if (have && qi < nq && g < gn && key >= lo && key <= pos) {
                        sc = dot[row] * a.scale;
                        if (a.cap > 0.f) sc = a.cap * tanhf(sc / a.cap);
                        if (a.dist_bias) sc += a.dist_bias[(size_t)(h0 + g) * a.L + min(pos - key, a.L - 1)];
                    }
                    Ps[row * KEYS + tid] = sc;
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
            const int nk = min(KEYS, pos_last + 1 - c0);
            for (int t = 0; t < nk; t += 4) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int key = c0 + t + j;
                    v[j] = (t + j < nk && tid < Dv)
                               ? to_float(vp[(((size_t)pg[t + j] * a.Hkv + kh) * BS + key % BS) * Dv + tid]) : 0.f;
                }
#pragma unroll
                for (int row = 0; row < ROWS; ++row) {
                    const float4 w = *reinterpret_cast<const float4*>(Ps + row * KEYS + t);
                    acc[row] = fmaf(w.x, v[0], fmaf(w.y, v[1], fmaf(w.z, v[2], fmaf(w.w, v[3], acc[row]))));
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int row = 0; row < ROWS; ++row) {
            const int qi = row / GP, g = row - qi * GP;
            if (qi >= nq || g >= gn || tid >= Dv) continue;
            const int h = h0 + g, n = n_first + qi;
            const float f = gate_factor<T>(a, n, h, tid) / run_sum[row];
            ((T*)a.out)[((size_t)n * a.Hq + h) * Dv + tid] = from_float<T>(acc[row] * f);
        }
    }
}

}  // namespace

extern "C" int sb_attention_bias(void* out, const void* q, const void* k_pool, const void* v_pool,
                                 const int* block_table, int table_width, const int* token_rows,
                                 const int* positions, const void* gate, long long gate_stride,
                                 const float* dist_bias, int L, int N, int Hq, int Hkv, int Dk, int Dv,
                                 int page_size, int window, float scale, float cap, int num_partitions,
                                 float* part_o, float* part_ml, int dtype, int gate_per_dim, int has_sink,
                                 float sink, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0,
               "attention_bias: %d query heads are no multiple of %d KV heads", Hq, Hkv);
    SB_REQUIRE(Dk >= 1 && Dk <= DMAX && Dv >= 1 && Dv <= 2 * THREADS,
               "attention_bias: head sizes %d (keys) and %d (values) must be at most %d", Dk, Dv, DMAX);
    SB_REQUIRE(page_size > 0 && table_width > 0, "attention_bias: bad page_size %d or table width %d", page_size,
               table_width);
    SB_REQUIRE(window >= 0, "attention_bias: window %d is negative", window);
    SB_REQUIRE(dist_bias == nullptr || L >= 1, "attention_bias: a bias table needs a length");
    SB_REQUIRE(N <= 65535, "attention_bias: %d tokens exceed one launch", N);
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 64 &&
                   (num_partitions == 1 || (part_o != nullptr && part_ml != nullptr)),
               "attention_bias: %d partitions (1 to 64; more than one needs scratch buffers)", num_partitions);
    if (N == 0) return 0;
    BiasAttnArgs a;
    a.out = out; a.q = q; a.k_pool = k_pool; a.v_pool = v_pool; a.block_table = block_table;
    a.table_width = table_width; a.token_rows = token_rows; a.positions = positions; a.gate = gate;
    a.gate_stride = gate_stride; a.dist_bias = dist_bias; a.L = L > 0 ? L : 1; a.Hq = Hq; a.Hkv = Hkv; a.Dk = Dk;
    a.Dv = Dv; a.BS = page_size; a.window = window; a.scale = scale; a.cap = cap;
    a.NP = num_partitions; a.part_o = part_o; a.part_ml = part_ml;
    a.gate_per_dim = gate_per_dim; a.has_sink = has_sink; a.sink = sink;
    dim3 grid(Hkv, N, num_partitions), rgrid(Hq, N);
    if (dtype == SB_F32) {
        sb::launch(bias_attention_kernel<float>, grid, dim3(THREADS), 0, stream, a);
        if (num_partitions > 1)
            sb::launch(attn_reduce_kernel<float>, rgrid, dim3(128), 0, stream, (float*)out, (const float*)part_o,
                       (const float*)part_ml, Hq, Dv, num_partitions);
    } else if (dtype == SB_BF16) {
        sb::launch(bias_attention_kernel<__nv_bfloat16>, grid, dim3(THREADS), 0, stream, a);
        if (num_partitions > 1)
            sb::launch(attn_reduce_kernel<__nv_bfloat16>, rgrid, dim3(128), 0, stream, (__nv_bfloat16*)out,
                       (const float*)part_o, (const float*)part_ml, Hq, Dv, num_partitions);
    } else {
        SB_REQUIRE(false, "attention_bias: unknown dtype %d", dtype);
    }
    SB_LAUNCH_CHECK();
}

// Prompt portions: a tile of consecutive tokens of a request per block (see bias_attention_tile_kernel).
// Returns SB_ERR_ARG for shapes the tile kernel does not take; `sb_attention_bias_tile_supports` says which.
extern "C" int sb_attention_bias_tile_supports(int Hq, int Hkv, int Dk, int Dv, int dtype) {
    const int vec = dtype == SB_BF16 ? 8 : 4;
    return Hq % Hkv == 0 && Dk % vec == 0 && Dk >= vec && Dk <= DMAX && Dv >= 1 && Dv <= THREADS;
}

extern "C" int sb_attention_bias_tile(void* out, const void* q, const void* k_pool, const void* v_pool,
                                      const int* block_table, int table_width, const int* seq_starts,
                                      const int* seq_rows, const int* seq_first_pos, int R, const void* gate,
                                      long long gate_stride, const float* dist_bias, int L, int N, int Hq, int Hkv,
                                      int Dk, int Dv, int page_size, int window, float scale, float cap, int dtype,
                                      int gate_per_dim, int has_sink, float sink, cudaStream_t stream) {
    SB_REQUIRE(sb_attention_bias_tile_supports(Hq, Hkv, Dk, Dv, dtype),
               "attention_bias_tile: heads %d/%d of %d (keys) and %d (values) are not served", Hq, Hkv, Dk, Dv);
    SB_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0, "attention_bias_tile: the key pool must be 16-byte aligned");
    SB_REQUIRE(page_size > 0 && table_width > 0 && window >= 0 && R >= 0, "attention_bias_tile: bad sizes");
    SB_REQUIRE(dist_bias == nullptr || L >= 1, "attention_bias_tile: a bias table needs a length");
    if (N == 0 || R == 0) return 0;
    const int G = Hq / Hkv;
    TileArgs ta;
    BiasAttnArgs& a = ta.b;
    a.out = out; a.q = q; a.k_pool = k_pool; a.v_pool = v_pool; a.block_table = block_table;
    a.table_width = table_width; a.token_rows = nullptr; a.positions = nullptr; a.gate = gate;
    a.gate_stride = gate_stride; a.dist_bias = dist_bias; a.L = L > 0 ? L : 1; a.Hq = Hq; a.Hkv = Hkv; a.Dk = Dk;
    a.Dv = Dv; a.BS = page_size; a.window = window; a.scale = scale; a.cap = cap; a.NP = 1; a.part_o = nullptr;
    a.part_ml = nullptr;
    a.gate_per_dim = gate_per_dim; a.has_sink = has_sink; a.sink = sink;
    ta.seq_starts = seq_starts; ta.seq_rows = seq_rows; ta.seq_first_pos = seq_first_pos; ta.R = R;
    ta.GP = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
    ta.QT = ROWS / ta.GP;
    const int tiles = (N + ta.QT - 1) / ta.QT + R;
    SB_REQUIRE(tiles <= 65535, "attention_bias_tile: %d tiles exceed one launch", tiles);
    const size_t smem = (size_t)ROWS * (Dk + KEYS) * sizeof(float);
    dim3 grid(Hkv, tiles);
    static sb::OncePerDevice once_f, once_b;
    if (dtype == SB_F32) {
        if (!once_f.flag()) {
            cudaFuncSetAttribute(bias_attention_tile_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            once_f.flag() = true;
        }
        sb::launch(bias_attention_tile_kernel<float>, grid, dim3(THREADS), smem, stream, ta);
    } else {
        if (!once_b.flag()) {
            cudaFuncSetAttribute(bias_attention_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            once_b.flag() = true;
        }
        sb::launch(bias_attention_tile_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, ta);
    }
    SB_LAUNCH_CHECK();
}
