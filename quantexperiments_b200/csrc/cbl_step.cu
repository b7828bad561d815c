// The kernels of a decode step that sit between the packed linears (Qwen2-style blocks): embedding rows,
// residual add + RMSNorm, rotary embedding + KV-cache write, grouped-query decode attention over the cache
// (position slices in parallel, then a merge), silu(gate) * up, the dense 16-bit output head for small
// batches, and greedy argmax.  They follow the arithmetic of the reference's batch-1 engine
// (shapequant/kernels/decode_e2e.py:63-309): fp32 residual stream, activations rounded to the model's
// 16-bit type between operations, biases added and silu * up multiplied in that type, cos / sin rounded
// to it.  Every kernel handles B sequences (grid dimension) so that the batched engine
// (shapequant/runtime_batch.py) shares them.
//
// All launches use programmatic stream serialization: a kernel may become resident while its predecessor
// drains and waits (griddepcontrol.wait) before it touches memory.
#include "cbl_common.cuh"

namespace {

template <int CLUSTER_X = 1, typename... KA, typename... A>
int step_launch(void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A... args) {
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CLUSTER_X;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = CLUSTER_X > 1 ? 2 : 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...));
    return cbl_check_launch();
}

__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }

// 8 values of a 16-byte vector of T as floats
template <typename T> __device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& w, float (&f)[8]) {
    const __half2* p = (const __half2*)&w;
#pragma unroll
    for (int i = 0; i < 4; i++) { const float2 v = __half22float2(p[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---------------------------------------------------------------------------------------- embedding rows
template <typename T>
__global__ void __launch_bounds__(256) k_embed(const T* __restrict__ E, const int64_t* __restrict__ tok, int64_t rows, int H,
                                               float* __restrict__ h) {
    pdl_enter();
    const int b = blockIdx.y;
    int64_t t = tok[b] % rows;
    if (t < 0) t += rows;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) h[(int64_t)b * H + i] = to_f(E[t * H + i]);
}

// ---------------------------------------------------------------------------------------- add + RMSNorm
// h[b] += add[b] (if add); x[b] = T(h[b] * rsqrt(mean(h[b]^2) + eps) * w).  One block per sequence.
template <typename T>
__global__ void __launch_bounds__(512) k_add_rmsnorm(float* __restrict__ h, const T* __restrict__ add, int64_t ld_add,
                                                     const T* __restrict__ w, float eps, int H, T* __restrict__ x) {
    pdl_enter();
    __shared__ float red[16];
    const int b = blockIdx.x, tid = threadIdx.x;
    float* hb = h + (int64_t)b * H;
    float ss = 0.f;
    for (int i = tid; i < H; i += blockDim.x) {
        float v = hb[i];
        if (add) { v += to_f(add[(int64_t)b * ld_add + i]); hb[i] = v; }
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid < 32) {
        float v = tid < (int)(blockDim.x >> 5) ? red[tid] : 0.f;
        v = warp_sum(v);
        if (tid == 0) red[0] = v;
    }
    __syncthreads();
    const float rstd = rsqrtf(red[0] / (float)H + eps);
    for (int i = tid; i < H; i += blockDim.x) x[(int64_t)b * H + i] = cbl_cvt_out<T>(hb[i] * rstd * to_f(w[i]));
}

// ---------------------------------------------------------------------------------------- rotary + cache write
// Row r of qkv ([rows, ld]: q heads | k heads | v heads) belongs to sequence seq(r) at position p(r):
// decode (pos != null): seq = r, p = pos[r]; prefill (pos == null): seq = seq0, p = pos0 + r.
// Blocks (head, row): heads 0..NH-1 rotate q into qo [rows, NH*HD]; heads NH..NH+NKV-1 rotate k and copy v
// (+ bias) into the caches: keys [seq][NKV][max_len][HD], values dimension-major [seq][NKV][HD][max_len] (the layout
// the attention kernel's tensor-core value product reads without a transpose).
template <typename T>
__global__ void __launch_bounds__(128) k_rope_kv(const T* __restrict__ qkv, int64_t ld, const T* __restrict__ bias,
                                                 const int32_t* __restrict__ pos, int pos0, int seq0, int NH, int NKV, int HD,
                                                 float theta, int max_len, T* __restrict__ qo, T* __restrict__ kc, T* __restrict__ vc) {
    pdl_enter();
    const int hd = blockIdx.x, r = blockIdx.y, i = threadIdx.x, half = HD >> 1;
    if (i >= half) return;
    const int p = pos ? pos[r] : pos0 + r;
    const int seq = pos ? r : seq0;
    if (p < 0 || p >= max_len) return;
    const float inv = 1.f / powf(theta, (2.f * (float)i) / (float)HD);
    const float ang = (float)p * inv;
    const float c = to_f(cbl_cvt_out<T>(cosf(ang))), s = to_f(cbl_cvt_out<T>(sinf(ang)));
    const T* row = qkv + (int64_t)r * ld;
    const int o = hd * HD;                                   // q | k share the column arithmetic up to NH + NKV heads
    auto in = [&](int col) {
        const T v = row[col];
        return bias ? to_f(cbl_cvt_out<T>(to_f(v) + to_f(bias[col]))) : to_f(v);
    };
    const float x1 = in(o + i), x2 = in(o + i + half);
    const T r1 = cbl_cvt_out<T>(x1 * c - x2 * s), r2 = cbl_cvt_out<T>(x2 * c + x1 * s);
    if (hd < NH) {
        T* q = qo + (int64_t)r * NH * HD + o;
        q[i] = r1;
        q[i + half] = r2;
    } else {
        const int kv = hd - NH;
        const int64_t co = (((int64_t)seq * NKV + kv) * max_len + p) * HD;
        kc[co + i] = r1;
        kc[co + i + half] = r2;
        const int ov = (NH + NKV + kv) * HD;
        const int64_t vo = ((int64_t)seq * NKV + kv) * HD * max_len + p;      // values are cached dimension-major: [seq][kv][HD][max_len]
        vc[vo + (int64_t)i * max_len] = cbl_cvt_out<T>(in(ov + i));
        vc[vo + (int64_t)(i + half) * max_len] = cbl_cvt_out<T>(in(ov + i + half));
    }
}

// ---------------------------------------------------------------------------------------- decode attention
// Flash-decoding on mma.sync tensor cores.  One block per (position slice, kv head, sequence); its four warps walk
// the slice independently, 32 positions at a time, each with its own online softmax.  Per 32 positions:
//   scores  S^T[head][pos] = Q[head][dim] . K^T: the group's REP (<= 8) query heads are the M side (rows 8..15 of the
//           16-row MMA are zero), 4 tiles of 8 positions the N side; a lane loads the K row of "its" position with four
//           16-byte loads (the dimension order inside an MMA is permuted the same way for Q and K, so no shuffles);
//   values  O[head][dim] += P[head][pos] . V[pos][dim]: the score accumulators ARE the A fragments of this product
//           (the positions of a score tile are chosen so that they line up), and because the value cache is stored
//           dimension-major a lane's B fragment is 16 contiguous bytes of a V^T row (8 positions of one dimension).
// K and V are read once for all heads of the group; nothing is staged in shared memory.  Every warp writes its running
// max, denominator and un-normalised output per head; k_attn_merge combines the 4 * nsplit partial results.
constexpr int ATT_WARPS = 4, ATT_THREADS = ATT_WARPS * 32;
constexpr int ATT_HD = 128;
constexpr int ATT_PART = ATT_HD + 4;       // floats per partial result: HD sums, max, denominator, 2 of padding (16-byte rows)

__host__ __device__ inline void att_slice(int L, int nsplit, int split, int& s0, int& s1) {
    int per = (L + nsplit - 1) / nsplit;
    per = (per + 31) / 32 * 32;
    s0 = split * per;
    s1 = s0 + per < L ? s0 + per : L;
}

template <typename T> __device__ __forceinline__ void att_mma(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void att_mma<__half>(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void att_mma<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t att_pack(float lo, float hi);
template <> __device__ __forceinline__ uint32_t att_pack<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *(const uint32_t*)&h;
}
template <> __device__ __forceinline__ uint32_t att_pack<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(const uint32_t*)&h;
}

template <typename T, int REP>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_slice(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                                                            const int32_t* __restrict__ pos, int NKV, int max_len, float scale,
                                                            float* __restrict__ part) {
    pdl_enter();
    constexpr int HD = ATT_HD;
    const int split = blockIdx.x, kv = blockIdx.y, b = blockIdx.z, nsplit = gridDim.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int NH = NKV * REP;
    // positions 0..pos[b] are in the cache (the step's own included); a position outside the cache (a caller that
    // stepped past max_len) is clamped, so that no read ever leaves the cache
    const int L = min(max(pos[b] + 1, 0), max_len);
    int s0, s1;
    att_slice(L, nsplit, split, s0, s1);
    // partial result of (this warp, head g): [HD sums | max | denominator]
    const int nparts = nsplit * ATT_WARPS;
    float* pout = part + ((((int64_t)b * NH + kv * REP + g) * nparts) + split * ATT_WARPS + warp) * ATT_PART;
    const bool head_ok = g < REP;
    if (s0 + 32 * warp >= s1) {                                      // nothing for this warp
        if (head_ok && t == 0) { pout[HD] = -3.0e38f; pout[HD + 1] = 0.f; }
        return;
    }
    // Q fragments of head g: k16-step s covers, for lane t, dimensions 32t + 8(s/2) + 4(s%2) + {0,1 | 2,3}
    uint32_t qa[8][2];
    {
        const uint32_t* qrow = (const uint32_t*)(q + ((int64_t)b * NH + kv * REP + (head_ok ? g : 0)) * HD);
#pragma unroll
        for (int s = 0; s < 8; s++) {
            const int d0 = 32 * t + 8 * (s >> 1) + 4 * (s & 1);
            qa[s][0] = head_ok ? __ldg(qrow + (d0 >> 1)) : 0u;
            qa[s][1] = head_ok ? __ldg(qrow + (d0 >> 1) + 1) : 0u;
        }
    }
    const T* kbase = kc + ((int64_t)b * NKV + kv) * max_len * HD + 32 * t;                  // + position * HD
    const T* vbase = vc + (((int64_t)b * NKV + kv) * HD + g) * max_len + 8 * t;             // + 8 j * max_len + p0
    float m = -3.0e38f, l = 0.f;
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; j++)
#pragma unroll
        for (int k = 0; k < 4; k++) o[j][k] = 0.f;
    for (int p0 = s0 + 32 * warp; p0 < s1; p0 += 32 * ATT_WARPS) {
        // ---- scores: tile u, column n <-> position p0 + 8 (n / 2) + 2 u + n % 2; this lane supplies column g and receives columns 2t, 2t + 1
        float sc[4][2];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int pk = p0 + 8 * (g >> 1) + 2 * u + (g & 1);
            uint4 kw[4];
#pragma unroll
            for (int c = 0; c < 4; c++) kw[c] = pk < s1 ? __ldg((const uint4*)(kbase + (int64_t)pk * HD) + c) : make_uint4(0, 0, 0, 0);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const uint4 w = kw[s >> 1];
                att_mma<T>(acc, qa[s][0], qa[s][1], (s & 1) ? w.z : w.x, (s & 1) ? w.w : w.y);
            }
            const int pc = p0 + 8 * t + 2 * u;                       // position of column 2t of tile u
            sc[u][0] = pc < s1 ? acc[0] * scale : -3.0e38f;
            sc[u][1] = pc + 1 < s1 ? acc[1] * scale : -3.0e38f;
        }
        // ---- online softmax of head g over the chunk (its 32 positions live in the four lanes t of this g)
        float cm = fmaxf(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])), fmaxf(fmaxf(sc[2][0], sc[2][1]), fmaxf(sc[3][0], sc[3][1])));
        cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 1));
        cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 2));
        const float mn = fmaxf(m, cm);
        const float rescale = __expf(m - mn);
        m = mn;
        float ps = 0.f;
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                sc[u][e] = sc[u][e] > -1.0e38f ? __expf(sc[u][e] - mn) : 0.f;
                ps += sc[u][e];
            }
        l = l * rescale + ps;
        // the probabilities of positions 8t..8t+3 / 8t+4..8t+7 are the A fragments of the two value MMAs
        const uint32_t pa0 = att_pack<T>(sc[0][0], sc[0][1]), pa2 = att_pack<T>(sc[1][0], sc[1][1]);
        const uint32_t pb0 = att_pack<T>(sc[2][0], sc[2][1]), pb2 = att_pack<T>(sc[3][0], sc[3][1]);
        // ---- values: dimension tile j = dimensions 8j..8j+7; this lane supplies dimension 8j + g, positions p0 + 8t..8t+7
#pragma unroll
        for (int j0 = 0; j0 < 16; j0 += 4) {
            uint4 vw[4];
#pragma unroll
            for (int j = 0; j < 4; j++) vw[j] = __ldg((const uint4*)(vbase + (int64_t)(8 * (j0 + j)) * max_len + p0));
#pragma unroll
            for (int j = 0; j < 4; j++) {
#pragma unroll
                for (int k = 0; k < 4; k++) o[j0 + j][k] *= rescale;
                att_mma<T>(o[j0 + j], pa0, pa2, vw[j].x, vw[j].y);
                att_mma<T>(o[j0 + j], pb0, pb2, vw[j].z, vw[j].w);
            }
        }
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (head_ok) {
#pragma unroll
        for (int j = 0; j < 16; j++) *(float2*)(pout + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (t == 0) { pout[HD] = m; pout[HD + 1] = l; }
    }
}

// out[b][head][:] = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) l_s.  One block per (head, sequence): the parts'
// weights are computed once (a thread per part), then every thread sums its output dimension; with many parts (few
// sequences: few blocks, pure latency) four groups of 128 threads each take every fourth part and their sums are
// added through shared memory.
constexpr int ATT_MAX_SPLITS = 512;
constexpr int ATT_MERGE_GROUPS = 4;
template <typename T, int G>
__global__ void __launch_bounds__(ATT_HD * G) k_attn_merge(const float* __restrict__ part, int nsplit, T* __restrict__ out) {
    pdl_enter();
    constexpr int HD = ATT_HD, NT = ATT_HD * G;                      // G groups of 128 threads
    __shared__ float s_w[ATT_MAX_SPLITS];
    __shared__ float s_red[NT / 32];
    __shared__ float s_num[G][HD];
    const int head = blockIdx.x, b = blockIdx.y, NH = gridDim.x, tid = threadIdx.x, d = tid & (HD - 1), grp = tid >> 7;
    const float* p = part + ((int64_t)b * NH + head) * nsplit * ATT_PART;
    float m = -3.0e38f;
    for (int s = tid; s < nsplit; s += NT) m = fmaxf(m, p[s * ATT_PART + HD]);
    m = warp_max(m);
    if ((tid & 31) == 0) s_red[tid >> 5] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int w = 1; w < NT / 32; w++) m = fmaxf(m, s_red[w]);
    __syncthreads();
    float den = 0.f;
    for (int s = tid; s < nsplit; s += NT) {
        const float l = p[s * ATT_PART + HD + 1];
        const float w = l > 0.f ? __expf(p[s * ATT_PART + HD] - m) : 0.f;
        s_w[s] = w;
        den += w * l;
    }
    den = warp_sum(den);
    if ((tid & 31) == 0) s_red[tid >> 5] = den;
    __syncthreads();
    den = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; w++) den += s_red[w];
    float num = 0.f;
#pragma unroll 8
    for (int s = grp; s < nsplit; s += G) {
        const float v = p[s * ATT_PART + d];
        num += s_w[s] != 0.f ? s_w[s] * v : 0.f;                  // a part without positions wrote no sums (whatever is there is ignored)
    }
    s_num[grp][d] = num;
    __syncthreads();
    if (grp == 0) {
#pragma unroll
        for (int q = 1; q < G; q++) num += s_num[q][d];
        out[((int64_t)b * NH + head) * HD + d] = cbl_cvt_out<T>(den > 0.f ? num / den : 0.f);
    }
}

// ---------------------------------------------------------------------------------------- silu(gate) * up
template <typename T>
__global__ void __launch_bounds__(256) k_silu_mul(const T* __restrict__ gu, int64_t ld, int I, T* __restrict__ out) {
    pdl_enter();
    const int b = blockIdx.y;
    const T* row = gu + (int64_t)b * ld;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < I; i += gridDim.x * blockDim.x) {
        const float a = to_f(row[i]);
        const float sl = to_f(cbl_cvt_out<T>(a / (1.f + __expf(-a))));       // silu and the product are rounded to the model type
        out[(int64_t)b * I + i] = cbl_cvt_out<T>(sl * to_f(row[I + i]));
    }
}

// ---------------------------------------------------------------------------------------- dense 16-bit head, B <= 8
// logits[b][v] = <W[v], x[b]>.  A warp per vocabulary row (persistent over rows), the row read with 16-byte
// loads, the B activation vectors in shared memory.  Streaming, HBM-bound.
constexpr int HEAD_BMAX = 8;
template <typename T, int B>
__global__ void __launch_bounds__(256) k_head(const T* __restrict__ W, const T* __restrict__ x, int V, int H, void* __restrict__ logits,
                                              int ldtype, int64_t ldl) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char s_raw[];
    T* s_x = (T*)s_raw;                                              // [B][H]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < B * H / 8; i += 256) ((uint4*)s_x)[i] = ((const uint4*)x)[i];
    __syncthreads();
    const int nvec = H / 8;
    for (int v = blockIdx.x * 8 + warp; v < V; v += gridDim.x * 8) {
        const uint4* wr = (const uint4*)(W + (int64_t)v * H);
        float acc[B];
#pragma unroll
        for (int b = 0; b < B; b++) acc[b] = 0.f;
        for (int c0 = 0; c0 < nvec; c0 += 32 * 4) {
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = c0 + u * 32 + lane;
                w[u] = c < nvec ? cbl_ldg_stream(wr + c) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = c0 + u * 32 + lane;
                if (c < nvec) {
                    float f[8];
                    unpack8<T>(w[u], f);
#pragma unroll
                    for (int b = 0; b < B; b++) {
                        float g[8];
                        unpack8<T>(((const uint4*)(s_x + (int64_t)b * H))[c], g);
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[b] += f[j] * g[j];
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            const float s = warp_sum(acc[b]);
            if (lane == 0) cbl_store_out(logits, ldtype, (int64_t)b * ldl + v, s);
        }
    }
}

// ---------------------------------------------------------------------------------------- block-32 embedding and head
// 4-bit block-32 embedding rows (shapequant/packed.py:33-36): h[b][i] = (nibble - 8) * scale[t][i / 32], even column in
// the low nibble.  Exact in fp32.
__global__ void __launch_bounds__(256) k_embed_q4(const uint8_t* __restrict__ Q, const __half* __restrict__ S, const int64_t* __restrict__ tok,
                                                  int64_t rows, int H, float* __restrict__ h) {
    pdl_enter();
    const int b = blockIdx.y;
    int64_t t = tok[b] % rows;
    if (t < 0) t += rows;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
        const uint8_t by = Q[t * (H >> 1) + (i >> 1)];
        const int n = (i & 1) ? (by >> 4) : (by & 15);
        h[(int64_t)b * H + i] = (float)(n - 8) * __half2float(S[t * (H >> 5) + (i >> 5)]);
    }
}

// 8-bit block-32 head (Q8_0-like, shapequant/packed.py:38-39): logits[b][v] = sum over blocks of scale * <q, x[b]>, on
// mma.sync tensor cores.  A warp owns 16 vocabulary rows; per block of 32 columns a lane loads 8 bytes of rows g and
// g + 8, turns the int8 weights into fp16 exactly (byte permute + magic-number subtract) and issues two m16n8k16 MMAs
// against the fp16 activations of up to 8 sequences (staged by cbl_prep_x: one power-of-two scale per sequence; in
// shared memory with a padded row stride), then adds scale * block sum to its fp32 accumulators.  Streaming, HBM-bound
// (8.5 bits per weight); the order of the columns inside an MMA is permuted identically for weights and activations.
constexpr int HQ_BMAX = 8;
__device__ __forceinline__ void hq_s8x4_to_h2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
    // bytes b0..b3 (signed) -> half2 {b0, b1}, {b2, b3}: fp16(1024 + (b ^ 0x80)) - 1152 = b exactly
    const uint32_t x = w ^ 0x80808080u;
    uint32_t p0, p1;
    asm("prmt.b32 %0, %1, %2, 0x7150;" : "=r"(p0) : "r"(x), "r"(0x64646464u));      // {x.b0, 0x64, x.b1, 0x64}
    asm("prmt.b32 %0, %1, %2, 0x7352;" : "=r"(p1) : "r"(x), "r"(0x64646464u));      // {x.b2, 0x64, x.b3, 0x64}
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));   // 1152
    const __half2 a = __hsub2(*(const __half2*)&p0, bias), c = __hsub2(*(const __half2*)&p1, bias);
    lo = *(const uint32_t*)&a;
    hi = *(const uint32_t*)&c;
}

__global__ void __launch_bounds__(256, 3) k_head_q8(const int8_t* __restrict__ Q, const __half* __restrict__ S, const __half* __restrict__ xp,
                                                 const float* __restrict__ xinv, int B, int V, int H, int Cpad, void* __restrict__ logits,
                                                 int ldtype, int64_t ldl) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char s_raw[];
    __half* s_x = (__half*)s_raw;                                    // [B + 1][H + 8] fp16; the last row is zero (sequences beyond B)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int xs = H + 8;                                            // padded row stride: the 8 rows of a fragment load hit different banks
    for (int i = tid; i < (B + 1) * (H / 8); i += 256) {
        const int r = i / (H / 8), c = i - r * (H / 8);
        *(uint4*)(s_x + r * xs + c * 8) = r < B ? *(const uint4*)(xp + (int64_t)r * Cpad + c * 8) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const int nblk = H >> 5;
    const bool vec_scales = (nblk % 8 == 0) && (((uintptr_t)S & 15) == 0);
    const uint4* xrow = (const uint4*)(s_x + (g < B ? g : B) * xs + 8 * t);       // + 4 * blk (uint4 units): columns 32 blk + 8 t .. + 8 of sequence g
    for (int v0 = (blockIdx.x * 8 + warp) * 16; v0 < V; v0 += gridDim.x * 128) {
        const int ra = min(v0 + g, V - 1), rb = min(v0 + g + 8, V - 1);
        const uint2* qa = (const uint2*)(Q + (int64_t)ra * H) + t;  // + 4 * blk (uint2 units)
        const uint2* qb = (const uint2*)(Q + (int64_t)rb * H) + t;
        const __half* sa = S + (int64_t)ra * nblk;
        const __half* sb = S + (int64_t)rb * nblk;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        constexpr int HU = 8;                                        // blocks in flight per lane: 16 eight-byte loads + their scales
        for (int k0 = 0; k0 < nblk; k0 += HU) {
            uint2 wa[HU], wb[HU];
            float fa[HU], fb[HU];
#pragma unroll
            for (int u = 0; u < HU; u++) {
                const bool ok = k0 + u < nblk;
                wa[u] = ok ? __ldg(qa + 4 * (k0 + u)) : make_uint2(0, 0);
                wb[u] = ok ? __ldg(qb + 4 * (k0 + u)) : make_uint2(0, 0);
            }
            if (vec_scales) {                                        // the 8 scales of a row = one 16-byte load (the same for the 4 lanes of a row)
                union { uint4 u; __half h[8]; } va, vb;
                va.u = __ldg((const uint4*)(sa + k0));
                vb.u = __ldg((const uint4*)(sb + k0));
#pragma unroll
                for (int u = 0; u < HU; u++) { fa[u] = __half2float(va.h[u]); fb[u] = __half2float(vb.h[u]); }
            } else {
#pragma unroll
                for (int u = 0; u < HU; u++) {
                    const bool ok = k0 + u < nblk;
                    fa[u] = ok ? __half2float(__ldg(sa + k0 + u)) : 0.f;
                    fb[u] = ok ? __half2float(__ldg(sb + k0 + u)) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < HU; u++) {
                if (k0 + u < nblk) {
                    const uint4 xv = xrow[4 * (k0 + u)];
                    uint32_t a0, a2, a1, a3, c0, c2, c1, c3;
                    hq_s8x4_to_h2x2(wa[u].x, a0, a2);                // row g,     columns 8t + {0,1 | 2,3}
                    hq_s8x4_to_h2x2(wb[u].x, a1, a3);                // row g + 8
                    hq_s8x4_to_h2x2(wa[u].y, c0, c2);                // columns 8t + {4,5 | 6,7}
                    hq_s8x4_to_h2x2(wb[u].y, c1, c3);
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
                    cbl_mma16816(d, a0, a1, a2, a3, xv.x, xv.y);
                    cbl_mma16816(d, c0, c1, c2, c3, xv.z, xv.w);
                    acc[0] += fa[u] * d[0];
                    acc[1] += fa[u] * d[1];
                    acc[2] += fb[u] * d[2];
                    acc[3] += fb[u] * d[3];
                }
            }
        }
        // d[0], d[1]: row g, sequences 2t, 2t + 1; d[2], d[3]: row g + 8
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int n = 2 * t + e;
            if (n < B) {
                if (v0 + g < V) cbl_store_out(logits, ldtype, (int64_t)n * ldl + v0 + g, acc[e] * xinv[n]);
                if (v0 + g + 8 < V) cbl_store_out(logits, ldtype, (int64_t)n * ldl + v0 + g + 8, acc[2 + e] * xinv[n]);
            }
        }
    }
}

// The 16-bit head for 2..8 sequences on mma.sync (the FMA kernel above is at the HBM roofline for one sequence but its
// arithmetic grows with the batch): a warp owns 16 vocabulary rows, per block of 32 columns a lane loads 16 bytes of
// rows g and g + 8 straight into the A fragments of two m16n8k16 MMAs (same column permutation for the activations,
// which sit in shared memory with a padded row stride; sequences beyond B read a zero row).
template <typename T> __device__ __forceinline__ void head_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void head_mma<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    cbl_mma16816(c, a0, a1, a2, a3, b0, b1);
}
template <> __device__ __forceinline__ void head_mma<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                                    uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__global__ void __launch_bounds__(256, 3) k_head_mma(const T* __restrict__ W, const T* __restrict__ x, int B, int V, int H, void* __restrict__ logits,
                                                     int ldtype, int64_t ldl) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char s_raw[];
    T* s_x = (T*)s_raw;                                              // [B + 1][H + 8]; the last row is zero
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int xs = H + 8;
    for (int i = tid; i < (B + 1) * (H / 8); i += 256) {
        const int r = i / (H / 8), c = i - r * (H / 8);
        *(uint4*)(s_x + r * xs + c * 8) = r < B ? *(const uint4*)(x + (int64_t)r * H + c * 8) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const int nblk = H >> 5;
    const uint4* xrow = (const uint4*)(s_x + (g < B ? g : B) * xs + 8 * t);
    for (int v0 = (blockIdx.x * 8 + warp) * 16; v0 < V; v0 += gridDim.x * 128) {
        const int ra = min(v0 + g, V - 1), rb = min(v0 + g + 8, V - 1);
        const uint4* qa = (const uint4*)(W + (int64_t)ra * H) + t;  // + 4 * blk: columns 32 blk + 8 t .. + 8
        const uint4* qb = (const uint4*)(W + (int64_t)rb * H) + t;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        constexpr int HU = 4;
        for (int k0 = 0; k0 < nblk; k0 += HU) {
            uint4 wa[HU], wb[HU];
#pragma unroll
            for (int u = 0; u < HU; u++) {
                const bool ok = k0 + u < nblk;
                wa[u] = ok ? cbl_ldg_stream(qa + 4 * (k0 + u)) : make_uint4(0, 0, 0, 0);
                wb[u] = ok ? cbl_ldg_stream(qb + 4 * (k0 + u)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < HU; u++) {
                if (k0 + u < nblk) {
                    const uint4 xv = xrow[4 * (k0 + u)];
                    head_mma<T>(acc, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
                    head_mma<T>(acc, wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int n = 2 * t + e;
            if (n < B) {
                if (v0 + g < V) cbl_store_out(logits, ldtype, (int64_t)n * ldl + v0 + g, acc[e]);
                if (v0 + g + 8 < V) cbl_store_out(logits, ldtype, (int64_t)n * ldl + v0 + g + 8, acc[2 + e]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------- greedy argmax
// tok[b] = first index of the largest logit of row b; pos[b] += 1 when pos is given.  A cluster of ARGMAX_CTAS
// thread blocks per row: every block reduces its share, block 0 collects the others' results through
// distributed shared memory.
constexpr int ARGMAX_CTAS = 8;
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__global__ void __launch_bounds__(1024) k_argmax(const void* __restrict__ logits, int ldtype, int64_t ldl, int V, int64_t* __restrict__ tok,
                                                 int32_t* __restrict__ pos) {
    pdl_enter();
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    __shared__ float s_bv;
    __shared__ int s_bi;
    const int b = blockIdx.y, tid = threadIdx.x, rank = blockIdx.x;             // the cluster spans blockIdx.x
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = rank * 1024 + tid; i < V; i += ARGMAX_CTAS * 1024) {
        const float v = cbl_load_in(logits, ldtype, (int64_t)b * ldl + i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    auto better = [](float v, int i, float w, int j) { return w > v || (w == v && j < i); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, best, o);
        const int j = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(best, bi, w, j)) { best = w; bi = j; }
    }
    if ((tid & 31) == 0) { s_v[tid >> 5] = best; s_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
        best = s_v[tid];
        bi = s_i[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, best, o);
            const int j = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(best, bi, w, j)) { best = w; bi = j; }
        }
        if (tid == 0) { s_bv = best; s_bi = bi; }
    }
    cluster_sync_all();                                              // every block's result is in its shared memory
    if (rank == 0 && tid < 32) {
        best = -INFINITY;
        bi = 0x7fffffff;
        if (tid < ARGMAX_CTAS) {
            uint32_t av, ai;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(av) : "r"(cbl_smem_u32(&s_bv)), "r"(tid));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ai) : "r"(cbl_smem_u32(&s_bi)), "r"(tid));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(best) : "r"(av) : "memory");
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(bi) : "r"(ai) : "memory");
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, best, o);
            const int j = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(best, bi, w, j)) { best = w; bi = j; }
        }
        if (tid == 0) {
            tok[b] = bi == 0x7fffffff ? 0 : bi;
            if (pos) pos[b] += 1;
        }
    }
    cluster_sync_all();                                              // no block leaves while block 0 may still read it
}

bool is16(int dt) { return dt == CBL_F16 || dt == CBL_BF16; }

}  // namespace

#define CBL_BY_TYPE(dt, ...)                                          \
    do {                                                              \
        if ((dt) == CBL_F16) { using T = __half; __VA_ARGS__; }       \
        else { using T = __nv_bfloat16; __VA_ARGS__; }                \
    } while (0)

extern "C" int cbl_embed_rows(const void* embed, int dtype, int64_t rows, int32_t H, const int64_t* tok, int32_t B, float* h, cbl_stream s) {
    if (!embed || !tok || !h || !is16(dtype) || rows < 1 || H < 1 || B < 0) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    if (B > 65535) return CBL_EUNSUPPORTED;
    const dim3 grid(cbl_ceil_div(H, 256) < 16 ? cbl_ceil_div(H, 256) : 16, B);
    CBL_BY_TYPE(dtype, return step_launch(k_embed<T>, grid, dim3(256), 0, (cudaStream_t)s, (const T*)embed, tok, rows, (int)H, h));
}

extern "C" int cbl_add_rmsnorm(float* h, const void* add, int64_t ld_add, const void* w, int dtype, float eps, int32_t B, int32_t H, void* x,
                               cbl_stream s) {
    if (!h || !w || !x || !is16(dtype) || H < 1 || B < 0) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    CBL_BY_TYPE(dtype, return step_launch(k_add_rmsnorm<T>, dim3(B), dim3(512), 0, (cudaStream_t)s, h, (const T*)add, ld_add, (const T*)w, eps,
                                          (int)H, (T*)x));
}

extern "C" int cbl_rope_kv(const void* qkv, int dtype, int64_t ld, const void* bias, const int32_t* pos, int32_t pos0, int32_t seq0,
                           int32_t rows, int32_t NH, int32_t NKV, int32_t HD, float theta, int32_t max_len, void* q_out, void* kc, void* vc,
                           cbl_stream s) {
    if (!qkv || !q_out || !kc || !vc || !is16(dtype) || rows < 0 || NH < 1 || NKV < 1 || max_len < 1) return CBL_EINVAL;
    if (HD < 2 || HD > 256 || (HD & 1)) return CBL_EUNSUPPORTED;
    if (rows == 0) return CBL_OK;
    if (rows > 65535) return CBL_EUNSUPPORTED;
    CBL_BY_TYPE(dtype, return step_launch(k_rope_kv<T>, dim3(NH + NKV, rows), dim3(128), 0, (cudaStream_t)s, (const T*)qkv, ld, (const T*)bias,
                                          pos, (int)pos0, (int)seq0, (int)NH, (int)NKV, (int)HD, theta, (int)max_len, (T*)q_out, (T*)kc,
                                          (T*)vc));
}

extern "C" size_t cbl_attn_decode_workspace_bytes(int32_t B, int32_t NH, int32_t nsplit) {
    if (B < 0 || NH < 0 || nsplit < 1) return 0;
    return (size_t)B * NH * nsplit * ATT_WARPS * ATT_PART * 4 + 16;
}

extern "C" int32_t cbl_attn_decode_max_splits(void) { return ATT_MAX_SPLITS / ATT_WARPS; }

template <typename T, int REP>
static int attn_launch(const void* q, const void* kc, const void* vc, const int32_t* pos, int B, int NKV, int max_len, float scale, void* out,
                       float* part, int nsplit, cudaStream_t st) {
    int rc = step_launch(k_attn_slice<T, REP>, dim3(nsplit, NKV, B), dim3(ATT_THREADS), 0, st, (const T*)q, (const T*)kc, (const T*)vc, pos,
                         NKV, max_len, scale, part);
    if (rc != CBL_OK) return rc;
    if (nsplit * ATT_WARPS > 32)
        return step_launch(k_attn_merge<T, ATT_MERGE_GROUPS>, dim3(NKV * REP, B), dim3(ATT_HD * ATT_MERGE_GROUPS), 0, st, (const float*)part,
                           nsplit * ATT_WARPS, (T*)out);
    return step_launch(k_attn_merge<T, 1>, dim3(NKV * REP, B), dim3(ATT_HD), 0, st, (const float*)part, nsplit * ATT_WARPS, (T*)out);
}

extern "C" int cbl_attn_decode(const void* q, const void* kc, const void* vc, const int32_t* pos, int dtype, int32_t B, int32_t NH, int32_t NKV,
                               int32_t HD, int32_t max_len, float scale, void* out, void* workspace, int32_t nsplit, cbl_stream s) {
    if (!q || !kc || !vc || !pos || !out || !workspace || !is16(dtype) || B < 0 || NH < 1 || NKV < 1 || nsplit < 1) return CBL_EINVAL;
    if (HD != ATT_HD || NH % NKV || NH / NKV > 8 || B > 65535 || nsplit > ATT_MAX_SPLITS / ATT_WARPS) return CBL_EUNSUPPORTED;
    if (max_len % 32) return CBL_EINVAL;                       // the value cache's rows are read 32 positions at a time
    if (B == 0) return CBL_OK;
    float* part = (float*)workspace;
    const cudaStream_t st = (cudaStream_t)s;
#define CBL_ATT(R) case R: CBL_BY_TYPE(dtype, return (attn_launch<T, R>(q, kc, vc, pos, B, NKV, max_len, scale, out, part, nsplit, st)))
    switch (NH / NKV) {
        CBL_ATT(1);
        CBL_ATT(2);
        CBL_ATT(3);
        CBL_ATT(4);
        CBL_ATT(5);
        CBL_ATT(6);
        CBL_ATT(7);
        default: CBL_ATT(8);
    }
#undef CBL_ATT
    return CBL_EUNSUPPORTED;
}

extern "C" int cbl_silu_mul(const void* gate_up, int dtype, int64_t ld, int32_t B, int32_t I, void* out, cbl_stream s) {
    if (!gate_up || !out || !is16(dtype) || B < 0 || I < 1) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    if (B > 65535) return CBL_EUNSUPPORTED;
    int gx = cbl_ceil_div(I, 256);
    const int cap = cbl_ceil_div(4 * cbl_sm_count(), B);
    if (gx > cap) gx = cap < 1 ? 1 : cap;
    CBL_BY_TYPE(dtype, return step_launch(k_silu_mul<T>, dim3(gx, B), dim3(256), 0, (cudaStream_t)s, (const T*)gate_up, ld, (int)I, (T*)out));
}

extern "C" int32_t cbl_head_gemv_max_batch(void) { return HEAD_BMAX; }

template <typename T, int B>
static int head_launch(const void* W, const void* x, int V, int H, void* logits, int ldtype, int64_t ldl, cudaStream_t st) {
    const size_t smem = (size_t)B * H * sizeof(T);
    if (smem > 200 * 1024) return CBL_EUNSUPPORTED;
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_head<T, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev] = true;
    }
    const int per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
    int grid = cbl_sm_count() * per_sm;
    if (grid > cbl_ceil_div(V, 8)) grid = cbl_ceil_div(V, 8);
    return step_launch(k_head<T, B>, dim3(grid), dim3(256), smem, st, (const T*)W, (const T*)x, V, H, logits, ldtype, ldl);
}

extern "C" int cbl_head_gemv(const void* W, const void* x, int dtype, int32_t B, int32_t V, int32_t H, void* logits, int ldtype, int64_t ldl,
                             cbl_stream s) {
    if (!W || !x || !logits || !is16(dtype) || V < 1 || H < 1 || B < 0) return CBL_EINVAL;
    if (ldtype != CBL_F32 && !is16(ldtype)) return CBL_EINVAL;
    if (B > HEAD_BMAX || H % 8) return CBL_EUNSUPPORTED;
    if (B == 0) return CBL_OK;
    const cudaStream_t st = (cudaStream_t)s;
    if (B >= 2 && H % 32 == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)x % 16) == 0 && (size_t)(B + 1) * (H + 8) * 2 <= 200 * 1024) {
        const size_t smem = (size_t)(B + 1) * (H + 8) * 2;
        static bool attr_mma[64] = {};
        int dev = 0;
        CBL_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_mma[dev]) {
            CBL_CUDA(cudaFuncSetAttribute(k_head_mma<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            CBL_CUDA(cudaFuncSetAttribute(k_head_mma<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_mma[dev] = true;
        }
        int grid = cbl_sm_count() * 4;
        if (grid > cbl_ceil_div(V, 128)) grid = cbl_ceil_div(V, 128);
        CBL_BY_TYPE(dtype, return step_launch(k_head_mma<T>, dim3(grid), dim3(256), smem, st, (const T*)W, (const T*)x, (int)B, (int)V, (int)H, logits,
                                              ldtype, ldl));
    }
#define CBL_HEAD(N) case N: CBL_BY_TYPE(dtype, return (head_launch<T, N>(W, x, V, H, logits, ldtype, ldl, st)))
    switch (B) {
        CBL_HEAD(1);
        CBL_HEAD(2);
        CBL_HEAD(3);
        CBL_HEAD(4);
        CBL_HEAD(5);
        CBL_HEAD(6);
        CBL_HEAD(7);
        default: CBL_HEAD(8);
    }
#undef CBL_HEAD
    return CBL_EUNSUPPORTED;
}

extern "C" int cbl_embed_rows_q4(const void* q, const void* scale, int64_t rows, int32_t H, const int64_t* tok, int32_t B, float* h, cbl_stream s) {
    if (!q || !scale || !tok || !h || rows < 1 || H < 32 || H % 32 || B < 0) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    if (B > 65535) return CBL_EUNSUPPORTED;
    const dim3 grid(cbl_ceil_div(H, 256) < 16 ? cbl_ceil_div(H, 256) : 16, B);
    return step_launch(k_embed_q4, grid, dim3(256), 0, (cudaStream_t)s, (const uint8_t*)q, (const __half*)scale, tok, rows, (int)H, h);
}

extern "C" size_t cbl_head_q8_scratch_bytes(int32_t B, int32_t H) { return cbl_prep_x_bytes(B, H, 1); }

extern "C" int32_t cbl_head_gemv_q8_max_batch(void) { return HQ_BMAX; }

extern "C" int cbl_head_gemv_q8(const void* q, const void* scale, const void* x, int dtype, int32_t B, int32_t V, int32_t H, void* logits, int ldtype,
                                int64_t ldl, void* scratch, cbl_stream s) {
    if (!q || !scale || !x || !logits || !scratch || !is16(dtype) || V < 1 || H < 32 || B < 0) return CBL_EINVAL;
    if (ldtype != CBL_F32 && !is16(ldtype)) return CBL_EINVAL;
    if (B > HQ_BMAX || H % 32) return CBL_EUNSUPPORTED;
    if (((uintptr_t)q % 16) || ((uintptr_t)scratch % 16)) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    const size_t smem = (size_t)(B + 1) * (H + 8) * 2;
    if (smem > 200 * 1024) return CBL_EUNSUPPORTED;
    const cudaStream_t st = (cudaStream_t)s;
    int rc = cbl_prep_x(x, dtype, B, H, H, nullptr, 1, scratch, s);          // fp16 [8][Cpad] + one power-of-two scale per sequence
    if (rc != CBL_OK) return rc;
    const int Cpad = (H + 511) / 512 * 512;
    const float* xinv = (const float*)((const __half*)scratch + (int64_t)8 * Cpad);
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_head_q8, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev] = true;
    }
    int grid = cbl_sm_count() * 4;
    if (grid > cbl_ceil_div(V, 128)) grid = cbl_ceil_div(V, 128);
    return step_launch(k_head_q8, dim3(grid), dim3(256), smem, st, (const int8_t*)q, (const __half*)scale, (const __half*)scratch, xinv, (int)B, (int)V,
                       (int)H, Cpad, logits, ldtype, ldl);
}

extern "C" int cbl_argmax(const void* logits, int ldtype, int64_t ldl, int32_t B, int32_t V, int64_t* tok, int32_t* pos, cbl_stream s) {
    if (!logits || !tok || V < 1 || B < 0 || (ldtype != CBL_F32 && !is16(ldtype))) return CBL_EINVAL;
    if (B == 0) return CBL_OK;
    if (B > 65535) return CBL_EUNSUPPORTED;
    return step_launch<ARGMAX_CTAS>(k_argmax, dim3(ARGMAX_CTAS, B), dim3(1024), 0, (cudaStream_t)s, logits, ldtype, ldl, (int)V, tok, pos);
}
