// gtb_seq_mixers.cuh -- mechanisms of the sequential (post-norm) layer style of the layer-list sequence models:
//   * RMS norm with a weight vector (plain or stored around zero), and the residual update x += norm(sublayer output)
//   * minGRU: an element-wise gated recurrence whose gates read only the current token (fp32 state per slot)
//   * softmax attention over a sliding window plus one mean key/value per block of tokens that has left the window, with a learned
//     sink in the denominator, tanh soft-capping of the scores, weighted per-head q/k norm, rotary positions (interleaved or split
//     pairs, frequencies from a host table), a sigmoid output gate, and keys/values that may come from another layer's cache
//   * PolyNorm activation, routed experts (softmax router with a choice correction, identity experts, squared-ReLU experts)
// Row kernels here serve every pass; the tiled kernels for prompt portions are in gtb_seq_mixers_tiled.cuh.
//
// Precision follows gtb_seq_kernels.cuh: everything below is fp32 except operands of matrix products and the K/V cache (type OT).
#pragma once
#include "gtb_seq_kernels.cuh"

namespace gtb {
namespace seq {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// maximum over the block; every thread gets the result.  red: 33 floats of shared memory.
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// four consecutive operand elements at once (the destination is 8- or 16-byte aligned)
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// ------------------------------------------------------------------------------------------------ norms
// out = x / sqrt(mean(x^2) + eps) * (one_plus + w[c]).  rows: optional gather (row index per output row).
template <typename OUT>
__global__ void __launch_bounds__(256) k_rmsnorm_weight(const float* __restrict__ x, int width, float eps, const float* __restrict__ w, int one_plus,
                                                        const int* __restrict__ rows, OUT* __restrict__ out, int ld_out) {
    __shared__ float red[33];
    const int o = blockIdx.x, r = rows ? rows[o] : o;
    const float* xr = x + (size_t)r * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)width + eps), base = one_plus ? 1.0f : 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)o * ld_out + c] = cvt<OUT>(xr[c] * sc * (base + w[c]));
}

// ------------------------------------------------------------------------------------------------ router
// One warp routes one row: s = softmax(z) over all n_out router outputs; the `top` outputs with the largest s + corr are chosen (ties to
// the lower index); sel_w holds their s (not renormalised).  s, ch: n_out floats of shared memory each.
__device__ __forceinline__ void route_row(const float* __restrict__ z, int n_out, const float* __restrict__ corr, int top, int* __restrict__ sel_idx,
                                          float* __restrict__ sel_w, float* s, float* ch, int lane) {
    float mx = -INFINITY;
    for (int i = lane; i < n_out; i += 32) mx = fmaxf(mx, z[i]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int i = lane; i < n_out; i += 32) { const float e = expf(z[i] - mx); s[i] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int i = lane; i < n_out; i += 32) { const float v = s[i] * inv; s[i] = v; ch[i] = v + (corr ? corr[i] : 0.0f); }
    __syncwarp();
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int i = lane; i < n_out; i += 32) { const float v = ch[i]; if (v > best) { best = v; arg = i; } }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
        }
        if (arg == 0x7fffffff) arg = 0;                  // every remaining choice score is -inf or NaN
        if (lane == 0) { sel_idx[k] = arg; sel_w[k] = s[arg]; ch[arg] = -INFINITY; }
        __syncwarp();
    }
}
// rows of router logits Z -> choices; shared memory: 2 n_out floats
__global__ void __launch_bounds__(32) k_moe_route(const float* __restrict__ Z, int ldz, int n_out, const float* __restrict__ corr, int top,
                                                  int* __restrict__ sel_idx, float* __restrict__ sel_w) {
    extern __shared__ float sm[];
    const int r = blockIdx.x;
    route_row(Z + (size_t)r * ldz, n_out, corr, top, sel_idx + (size_t)r * top, sel_w + (size_t)r * top, sm, sm + n_out, threadIdx.x);
}
// The router of the NEXT sublayer inside the residual update (few rows): what k_postnorm_add appends when it is given a router
struct RouteNext {
    const bf16* w;             // [n_out][ldw] router matrix, or null: no routing here
    int ldw, n_out, top;
    const float* corr;
    int* sel_idx;              // [rows][top]
    float* sel_w;
};

// router logits of row r from its new stream values sx [width] (fp32, shared memory) -- a warp per output -- and the row's choices
__device__ __forceinline__ void postnorm_route(const RouteNext& rn, float* sx, int width, int r) {
    float* sl = sx + width;              // [n_out] logits, then [n_out] scores and [n_out] choice scores
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    for (int j = wid; j < rn.n_out; j += nw) {
        const bf16* wr = rn.w + (size_t)j * rn.ldw;
        float a = 0.0f;
        const int w8 = width & ~7;                   // rows of the router matrix start on 16-byte boundaries: eight weights per load
        for (int c = lane * 8; c < w8; c += 256) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + c));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a = fmaf(sx[c + 2 * i], __uint_as_float(ww[i] << 16), a);
                a = fmaf(sx[c + 2 * i + 1], __uint_as_float(ww[i] & 0xffff0000u), a);
            }
        }
        for (int c = w8 + lane; c < width; c += 32) a = fmaf(sx[c], __bfloat162float(wr[c]), a);
        a = warp_sum(a);
        if (lane == 0) sl[j] = a;
    }
    __syncthreads();
    if (wid == 0) route_row(sl, rn.n_out, rn.corr, rn.top, rn.sel_idx + (size_t)r * rn.top, rn.sel_w + (size_t)r * rn.top, sl + rn.n_out, sl + 2 * rn.n_out, lane);
}

// Residual update of the post-norm style: y = Y (+ wid * x, the share of identity experts: pairs of sel_idx that are >= n_experts),
// x += y / sqrt(mean(y^2) + eps) * (1 + w); the new stream is also written as the operand of the next matrix product.
// Grouped experts: Y = null and the row's sublayer output is the sum of rows pair_dst[r * top + k] >= 0 of Yg (in order of k).
constexpr int PN_MAX_TOP = 64, PN_KEEP = 4;
template <typename OT>
__global__ void __launch_bounds__(256) k_postnorm_add(const float* __restrict__ Y, int width, float eps, const float* __restrict__ w,
                                                      const int* __restrict__ sel_idx, const float* __restrict__ sel_w, int top, int n_experts,
                                                      const float* __restrict__ Yg, const int* __restrict__ pair_dst,
                                                      float* __restrict__ x, OT* __restrict__ op, int ld_op, RouteNext rn) {
    __shared__ float red[33];
    __shared__ int sdst[PN_MAX_TOP];
    extern __shared__ float srt[];       // routing: the new stream row [width], logits [n_out], two work arrays [n_out]
    const int r = blockIdx.x;
    float wid = 0.0f;
    if (sel_idx)
        for (int k = 0; k < top; k++)
            if (sel_idx[(size_t)r * top + k] >= n_experts) wid += sel_w[(size_t)r * top + k];
    if (!Y && threadIdx.x < top) sdst[threadIdx.x] = pair_dst[(size_t)r * top + threadIdx.x];
    __syncthreads();
    auto sub = [&](int c) {
        if (Y) return Y[(size_t)r * width + c];
        float a = 0.0f;
        for (int k = 0; k < top; k++)
            if (sdst[k] >= 0) a += Yg[(size_t)sdst[k] * width + c];
        return a;
    };
    float* xr = x + (size_t)r * width;
    float ss = 0.0f;
    if (width % 4 == 0 && width <= 4 * PN_KEEP * (int)blockDim.x && ld_op % 4 == 0) {
        // rows of up to 4 * PN_KEEP * blockDim.x values stay in registers between the two passes: every input is read once, 16 bytes at a time
        float4 vx[PN_KEEP], vy[PN_KEEP];
#pragma unroll
        for (int i = 0; i < PN_KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) {
                vx[i] = *reinterpret_cast<const float4*>(xr + c);
                float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (Y) y = *reinterpret_cast<const float4*>(Y + (size_t)r * width + c);
                else
                    for (int k = 0; k < top; k++)
                        if (sdst[k] >= 0) { const float4 t4 = *reinterpret_cast<const float4*>(Yg + (size_t)sdst[k] * width + c); y.x += t4.x; y.y += t4.y; y.z += t4.z; y.w += t4.w; }
                y.x = fmaf(wid, vx[i].x, y.x); y.y = fmaf(wid, vx[i].y, y.y); y.z = fmaf(wid, vx[i].z, y.z); y.w = fmaf(wid, vx[i].w, y.w);
                vy[i] = y;
                ss += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
            }
        }
        ss = block_sum(ss, red);
        const float sc = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int i = 0; i < PN_KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) {
                const float4 g = *reinterpret_cast<const float4*>(w + c);
                const float4 xn = make_float4(vx[i].x + vy[i].x * sc * (1.0f + g.x), vx[i].y + vy[i].y * sc * (1.0f + g.y),
                                              vx[i].z + vy[i].z * sc * (1.0f + g.z), vx[i].w + vy[i].w * sc * (1.0f + g.w));
                *reinterpret_cast<float4*>(xr + c) = xn;
                store4(op + (size_t)r * ld_op + c, xn.x, xn.y, xn.z, xn.w);
                if (rn.w) { srt[c] = xn.x; srt[c + 1] = xn.y; srt[c + 2] = xn.z; srt[c + 3] = xn.w; }
            }
        }
        if (rn.w) postnorm_route(rn, srt, width, r);
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = fmaf(wid, xr[c], sub(c)); ss += v * v; }
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float xo = xr[c], v = fmaf(wid, xo, sub(c));
        const float xn = xo + v * sc * (1.0f + w[c]);
        xr[c] = xn;
        op[(size_t)r * ld_op + c] = cvt<OT>(xn);
        if (rn.w) srt[c] = xn;
    }
    if (rn.w) postnorm_route(rn, srt, width, r);
}

// ------------------------------------------------------------------------------------------------ minGRU
struct GruBranch {
    int width;
    int z_off, x_off, g_off;     // columns of the update gate, the candidate's pre-activation and the output gate in the projection buffer
    int a_off;                   // column of the output in the out-projection operand
};
// candidate of the recurrence: u + 1/2 on the non-negative side, logistic(u) below (continuous, positive)
__device__ __forceinline__ float gru_candidate(float u) { return u >= 0.0f ? u + 0.5f : sigmoidf_(u); }

// S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, z = logistic(P_z), c = candidate(P_x); out_t = S_t * silu(P_g).  One thread per
// (segment, channel) walks the segment's rows from the slot's state; the loads of eight rows are issued before their chain starts.
template <typename OT>
__global__ void __launch_bounds__(128) k_mingru(PassTables t, GruBranch b, const float* __restrict__ P, int ldp, float* __restrict__ state,
                                                OT* __restrict__ out, int ld_out) {
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= b.width) return;
    const int slot = t.seg_slot[s], row0 = t.seg_row0[s], len = t.seg_len[s];
    float* sp = state + (size_t)slot * b.width + c;
    float S = *sp;
    for (int n0 = 0; n0 < len; n0 += 8) {
        float z[8], u[8], g[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < len) {
                const float* p = P + (size_t)(row0 + n0 + i) * ldp;
                z[i] = p[b.z_off + c]; u[i] = p[b.x_off + c]; g[i] = p[b.g_off + c];
            }
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < len) {
                const float zz = sigmoidf_(z[i]);
                S = (1.0f - zz) * S + zz * gru_candidate(u[i]);
                out[(size_t)(row0 + n0 + i) * ld_out + b.a_off + c] = cvt<OT>(S * g[i] * sigmoidf_(g[i]));
            }
    }
    if (!t.slots[slot].stopped) *sp = S;
}

// Prompt portions: the recurrence is linear in S, so a chunk of C rows is the map S -> A S + B with A = prod (1 - z), B = the chunk run
// from zero.  k_mingru_chunk computes (A, B) of every chunk in parallel; k_mingru_chunk_out folds the maps of the chunks before its own
// (a few dozen multiply-adds) onto the slot's state, reruns its chunk from there and writes the outputs; k_mingru_store then moves the
// end state of every segment into its slot.  AB [chunk][2][width]; chunks are numbered segment by segment.
__device__ __forceinline__ bool gru_find_chunk(const PassTables& t, int S, int C, int idx, int& seg, int& c, int& first) {
    first = 0;
    for (int s = 0; s < S; s++) {
        const int n = (t.seg_len[s] + C - 1) / C;
        if (idx < first + n) { seg = s; c = idx - first; return true; }
        first += n;
    }
    return false;
}
__global__ void __launch_bounds__(128) k_mingru_chunk(PassTables t, GruBranch b, const float* __restrict__ P, int ldp, int S, int C, float* __restrict__ AB) {
    int seg, ck, first;
    if (!gru_find_chunk(t, S, C, blockIdx.x, seg, ck, first)) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= b.width) return;
    const int row0 = t.seg_row0[seg] + ck * C, L = min(C, t.seg_len[seg] - ck * C);
    float A = 1.0f, B = 0.0f;
    for (int n0 = 0; n0 < L; n0 += 8) {
        float z[8], u[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < L) { const float* p = P + (size_t)(row0 + n0 + i) * ldp; z[i] = p[b.z_off + c]; u[i] = p[b.x_off + c]; }
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < L) {
                const float zz = sigmoidf_(z[i]);
                A *= 1.0f - zz;
                B = (1.0f - zz) * B + zz * gru_candidate(u[i]);
            }
    }
    AB[((size_t)blockIdx.x * 2) * b.width + c] = A;
    AB[((size_t)blockIdx.x * 2 + 1) * b.width + c] = B;
}
template <typename OT>
__global__ void __launch_bounds__(128) k_mingru_chunk_out(PassTables t, GruBranch b, const float* __restrict__ P, int ldp, int S, int C,
                                                          float* __restrict__ AB, const float* __restrict__ state, OT* __restrict__ out, int ld_out) {
    int seg, ck, first;
    if (!gru_find_chunk(t, S, C, blockIdx.x, seg, ck, first)) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= b.width) return;
    const int slot = t.seg_slot[seg], len = t.seg_len[seg];
    const int row0 = t.seg_row0[seg] + ck * C, L = min(C, len - ck * C);
    float Sx = state[(size_t)slot * b.width + c];
    for (int k = 0; k < ck; k++) Sx = fmaf(AB[((size_t)(first + k) * 2) * b.width + c], Sx, AB[((size_t)(first + k) * 2 + 1) * b.width + c]);
    for (int n0 = 0; n0 < L; n0 += 8) {
        float z[8], u[8], g[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < L) {
                const float* p = P + (size_t)(row0 + n0 + i) * ldp;
                z[i] = p[b.z_off + c]; u[i] = p[b.x_off + c]; g[i] = p[b.g_off + c];
            }
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (n0 + i < L) {
                const float zz = sigmoidf_(z[i]);
                Sx = (1.0f - zz) * Sx + zz * gru_candidate(u[i]);
                out[(size_t)(row0 + n0 + i) * ld_out + b.a_off + c] = cvt<OT>(Sx * g[i] * sigmoidf_(g[i]));
            }
    }
    // Every chunk of the segment reads the slot's state, so it is not overwritten here: a segment's last chunk leaves the end state in
    // its own B entry (which no chunk folds) and k_mingru_store moves it to the slot afterwards.
    if ((ck + 1) * C >= len) AB[((size_t)blockIdx.x * 2 + 1) * b.width + c] = Sx;
}
__global__ void __launch_bounds__(128) k_mingru_store(PassTables t, GruBranch b, int S, int C, const float* __restrict__ AB, float* __restrict__ state) {
    const int seg = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= b.width) return;
    int last = -1;
    for (int s = 0; s <= seg; s++) last += (t.seg_len[s] + C - 1) / C;
    const int slot = t.seg_slot[seg];
    if (!t.slots[slot].stopped) state[(size_t)slot * b.width + c] = AB[((size_t)last * 2 + 1) * b.width + c];
}

// ------------------------------------------------------------------------------------------------ softmax attention
struct SoftAttn {
    int heads, kv_heads, dim, vdim;
    float scale, eps, softcap;   // softcap 0: scores are not capped
    int qk_norm;                 // 0: none, 1: unit RMS per head, 2: unit RMS times a weight vector shared by the heads, 3: one RMS norm over the
                                 // whole q (k) projection with a weight per entry; its scales come from qk_sc [rows][2] (k_proj_rms)
    const float *q_norm, *k_norm;
    int rot_dims, rot_layout;    // layout 0: pairs (i, i + rot_dims/2); 1: pairs (2i, 2i + 1)
    const float* inv_freq;       // [rot_dims / 2]
    int window, pool;            // window 0: every earlier token; pool 0: no pooled blocks
    const float* sink;           // [heads] or null
    int gate;                    // 0: none, 1: silu, 2: logistic, 3: logistic of one number per head (column g_off + head)
    int q_off, k_off, v_off, g_off, a_off;
    int k_ld, v_ld;              // row strides of the key / value cache in elements; 0: packed (kv_heads * dim, kv_heads * vdim)
    int own_kv;                  // 0: keys and values are another layer's cache (nothing is projected or appended here)
    int max_ctx, max_blocks;
    int maps;                    // 0 / 1: one score map per head; 2: two query parts per head and two key parts per K/V head ([part 1 | part 2]),
                                 // each (head, part) an attention of its own over the head's values.  Kernels index "query units" heads * maps
    int chunk;                   // > 0: a query sees only keys of its own chunk of positions
    float out_scale;             // weight of the output (0 counts as 1)
    const float* qk_sc;          // qk_norm 3
};
__host__ __device__ __forceinline__ int sa_maps(const SoftAttn& b) { return b.maps > 1 ? b.maps : 1; }

// q (and k): per-head norm, rotary positions; q in place (fp32), k and v appended to the slot's cache.
template <typename OT>
__global__ void __launch_bounds__(128) k_sattn_prep(PassTables t, SoftAttn b, float* __restrict__ P, int ldp, OT* __restrict__ kc, OT* __restrict__ vc) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    float* p = P + (size_t)r * ldp;
    const size_t crow = (size_t)slot * b.max_ctx + pos;
    const int M = sa_maps(b), nq = b.heads * M, nk = b.own_kv ? b.kv_heads * M : 0, nkv = b.own_kv ? b.kv_heads : 0, half = b.rot_dims / 2;
    const float fpos = (float)pos;
    for (int u = blockIdx.y * nw + wid; u < nq + nk + nkv; u += gridDim.y * nw) {
        if (u < nq + nk) {
            const bool is_q = u < nq;
            const int hu = is_q ? u : u - nq;
            float* v = p + (is_q ? b.q_off : b.k_off) + hu * b.dim;
            OT* dst = is_q ? nullptr : kc + crow * (size_t)(b.kv_heads * M * b.dim) + (size_t)hu * b.dim;
            const float* wn = b.qk_norm == 2 ? (is_q ? b.q_norm : b.k_norm) : b.qk_norm == 3 ? (is_q ? b.q_norm : b.k_norm) + (size_t)hu * b.dim : nullptr;
            float sc = 1.0f;
            if (b.qk_norm == 3) sc = b.qk_sc[(size_t)r * 2 + (is_q ? 0 : 1)];
            else if (b.qk_norm) {
                float ss = 0.0f;
                for (int i = lane; i < b.dim; i += 32) ss += v[i] * v[i];
                ss = warp_sum(ss);
                sc = 1.0f / sqrtf(ss / (float)b.dim + b.eps);
            }
            for (int pr = lane; pr < half; pr += 32) {
                const int i0 = b.rot_layout ? 2 * pr : pr, i1 = b.rot_layout ? 2 * pr + 1 : pr + half;
                const float a = v[i0] * sc * (wn ? wn[i0] : 1.0f), c = v[i1] * sc * (wn ? wn[i1] : 1.0f);
                float sn, cs;
                sincosf(fpos * b.inv_freq[pr], &sn, &cs);
                const float ra = a * cs - c * sn, rc = c * cs + a * sn;
                if (is_q) { v[i0] = ra; v[i1] = rc; } else { dst[i0] = cvt<OT>(ra); dst[i1] = cvt<OT>(rc); }
            }
            for (int i = b.rot_dims + lane; i < b.dim; i += 32) {
                const float a = v[i] * sc * (wn ? wn[i] : 1.0f);
                if (is_q) v[i] = a; else dst[i] = cvt<OT>(a);
            }
        } else {
            const int g = u - nq - nk;
            const float* v = p + b.v_off + g * b.vdim;
            OT* dst = vc + crow * (size_t)(b.kv_heads * b.vdim) + (size_t)g * b.vdim;
            for (int i = lane; i < b.vdim; i += 32) dst[i] = cvt<OT>(v[i]);
        }
    }
}

// A row whose position completes a block of `pool` tokens writes the block's mean key and mean value (of the cache's contents, summed
// in fp32) to the pooled cache pk / pv [n_slots][max_blocks][kv_heads * dim|vdim] (fp32).  Runs after every row of the pass is appended.
template <typename OT>
__global__ void __launch_bounds__(128) k_pool_update(PassTables t, SoftAttn b, const OT* __restrict__ kc, const OT* __restrict__ vc,
                                                     float* __restrict__ pk, float* __restrict__ pv) {
    const int r = blockIdx.x;
    const int slot = t.seg_slot[t.row_seg[r]], pos = t.row_pos[r];
    if ((pos + 1) % b.pool != 0) return;
    const int blk = pos / b.pool;
    const size_t kld = (size_t)b.kv_heads * b.dim, vld = (size_t)b.kv_heads * b.vdim;
    const OT* ks = kc + ((size_t)slot * b.max_ctx + (size_t)blk * b.pool) * kld;
    const OT* vs = vc + ((size_t)slot * b.max_ctx + (size_t)blk * b.pool) * vld;
    const float inv = 1.0f / (float)b.pool;
    // four partial sums per element: four loads in flight instead of a chain of `pool` dependent ones
    for (int e = threadIdx.x; e < (int)kld; e += blockDim.x) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        int i = 0;
        for (; i + 3 < b.pool; i += 4) {
            a0 += ldf<OT>(ks + (size_t)i * kld + e); a1 += ldf<OT>(ks + (size_t)(i + 1) * kld + e);
            a2 += ldf<OT>(ks + (size_t)(i + 2) * kld + e); a3 += ldf<OT>(ks + (size_t)(i + 3) * kld + e);
        }
        for (; i < b.pool; i++) a0 += ldf<OT>(ks + (size_t)i * kld + e);
        pk[((size_t)slot * b.max_blocks + blk) * kld + e] = ((a0 + a1) + (a2 + a3)) * inv;
    }
    for (int e = threadIdx.x; e < (int)vld; e += blockDim.x) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        int i = 0;
        for (; i + 3 < b.pool; i += 4) {
            a0 += ldf<OT>(vs + (size_t)i * vld + e); a1 += ldf<OT>(vs + (size_t)(i + 1) * vld + e);
            a2 += ldf<OT>(vs + (size_t)(i + 2) * vld + e); a3 += ldf<OT>(vs + (size_t)(i + 3) * vld + e);
        }
        for (; i < b.pool; i++) a0 += ldf<OT>(vs + (size_t)i * vld + e);
        pv[((size_t)slot * b.max_blocks + blk) * vld + e] = ((a0 + a1) + (a2 + a3)) * inv;
    }
}

__device__ __forceinline__ float soft_cap(float s, float cap) { return cap > 0.0f ? cap * tanhf(s / cap) : s; }
// keys a query at `pos` sees: pooled blocks 0 .. nb-1 (those that end at or before pos - window), then tokens lo .. pos
__device__ __forceinline__ void sattn_range(const SoftAttn& b, int pos, int& lo, int& nb) {
    lo = b.window > 0 ? max(0, pos - b.window + 1) : 0;
    if (b.chunk > 0) lo = max(lo, pos / b.chunk * b.chunk);
    nb = (b.window > 0 && b.pool > 0 && pos - b.window + 1 >= b.pool) ? (pos - b.window + 1) / b.pool : 0;
}

// Online softmax of one (row, query head) over the keys n_lo .. n_hi-1 of the list [pooled blocks | window tokens], in tiles of
// blockDim.x keys: a thread scores one key of the tile, then the threads turn to the value channels (vdim <= 4 * blockDim.x).
// m, l: running maximum and denominator (in / out); acc: this thread's value channels.  sm: dim + blockDim.x + 33 floats.
template <typename OT>
__device__ __forceinline__ void sattn_sweep(const PassTables& t, const SoftAttn& b, const float* __restrict__ P, int ldp, const OT* __restrict__ kc,
                                            const OT* __restrict__ vc, const float* __restrict__ pk, const float* __restrict__ pv, float* sm,
                                            int r, int h, int n_lo, int n_hi, int lo, int nb, float& m, float& l, float (&acc)[4]) {
    float* sq = sm;                 // [dim]
    float* swt = sm + b.dim;        // [blockDim.x]
    float* red = swt + blockDim.x;  // [33]
    const int M = sa_maps(b), g = (h / M) / (b.heads / b.kv_heads), ku = g * M + h % M, slot = t.seg_slot[t.row_seg[r]];      // h: query unit
    const float* q = P + (size_t)r * ldp + b.q_off + h * b.dim;
    for (int i = threadIdx.x; i < b.dim; i += blockDim.x) sq[i] = q[i];
    const size_t kld = b.k_ld ? (size_t)b.k_ld : (size_t)b.kv_heads * M * b.dim, vld = b.v_ld ? (size_t)b.v_ld : (size_t)b.kv_heads * b.vdim;
    const OT* kbase = kc + (size_t)slot * b.max_ctx * kld + (size_t)ku * b.dim;
    const OT* vbase = vc + (size_t)slot * b.max_ctx * vld + (size_t)g * b.vdim;
    const float* pkb = pk ? pk + (size_t)slot * b.max_blocks * kld + (size_t)ku * b.dim : nullptr;
    const float* pvb = pv ? pv + (size_t)slot * b.max_blocks * vld + (size_t)g * b.vdim : nullptr;
    const bool kvec = b.dim % 8 == 0 && kld % 8 == 0;
    __syncthreads();
    for (int n0 = n_lo; n0 < n_hi; n0 += blockDim.x) {
        const int n = n0 + threadIdx.x;
        float s = -INFINITY;
        if (n < n_hi) {
            const float d = n < nb ? key_dot(sq, pkb + (size_t)n * kld, b.dim, b.dim % 4 == 0) : key_dot(sq, kbase + (size_t)(lo + n - nb) * kld, b.dim, kvec);
            s = soft_cap(d * b.scale, b.softcap);
        }
        const float mn = fmaxf(m, block_max(s, red));
        const float corr = m == -INFINITY ? 0.0f : expf(m - mn);
        const float pw = n < n_hi ? expf(s - mn) : 0.0f;
        swt[threadIdx.x] = pw;
        l = l * corr + block_sum(pw, red);               // (its barriers also publish swt)
        m = mn;
        const int nj = min((int)blockDim.x, n_hi - n0);
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int c = threadIdx.x + cc * blockDim.x;
            if (c < b.vdim) {
                float a = acc[cc] * corr;
                for (int jj = 0; jj < nj; jj++) {
                    const int nn = n0 + jj;
                    const float v = nn < nb ? pvb[(size_t)nn * vld + c] : ldf<OT>(vbase + (size_t)(lo + nn - nb) * vld + c);
                    a = fmaf(swt[jj], v, a);
                }
                acc[cc] = a;
            }
        }
        __syncthreads();
    }
}
template <typename OT>
__device__ __forceinline__ void sattn_store(const SoftAttn& b, const float* __restrict__ P, int ldp, int r, int h, float inv, const float (&acc)[4],
                                            OT* __restrict__ out, int ld_out) {
    if (b.out_scale != 0.0f) inv *= b.out_scale;
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
        const int c = threadIdx.x + cc * blockDim.x;
        if (c < b.vdim) {
            float o = acc[cc] * inv;
            if (b.gate) {
                const float gt = P[(size_t)r * ldp + b.g_off + (b.gate == 3 ? h / sa_maps(b) : h * b.vdim + c)];
                o *= b.gate >= 2 ? sigmoidf_(gt) : gt * sigmoidf_(gt);
            }
            out[(size_t)r * ld_out + b.a_off + h * b.vdim + c] = cvt<OT>(o);
        }
    }
}

// One CTA per (row, query head) over all of the row's keys.  The running maximum starts at the sink and the denominator at 1
// (= exp(sink - sink)), so the sink counts once and no tile meets an empty history.
template <typename OT, typename OUT = OT>
__global__ void __launch_bounds__(128) k_sattn(PassTables t, SoftAttn b, const float* __restrict__ P, int ldp, const OT* __restrict__ kc, const OT* __restrict__ vc,
                                               const float* __restrict__ pk, const float* __restrict__ pv, OUT* __restrict__ out, int ld_out) {
    extern __shared__ float sm[];
    const int r = blockIdx.x, h = blockIdx.y, pos = t.row_pos[r];
    int lo, nb;
    sattn_range(b, pos, lo, nb);
    float m = b.sink ? b.sink[h / sa_maps(b)] : -INFINITY, l = b.sink ? 1.0f : 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    sattn_sweep<OT>(t, b, P, ldp, kc, vc, pk, pv, sm, r, h, 0, nb + pos - lo + 1, lo, nb, m, l, acc);
    sattn_store<OUT>(b, P, ldp, r, h, 1.0f / l, acc, out, ld_out);
}

// Decode rows: the keys of a (row, head) are split over gridDim.z CTAs in ranges of whole 128-key tiles; each leaves its running maximum,
// denominator and unnormalised value sum in part [split][R][heads][vdim + 2] (an empty range: maximum -inf), k_sattn_join folds the splits
// and the sink in order.
template <typename OT>
__global__ void __launch_bounds__(128) k_sattn_split(PassTables t, SoftAttn b, const float* __restrict__ P, int ldp, const OT* __restrict__ kc,
                                                     const OT* __restrict__ vc, const float* __restrict__ pk, const float* __restrict__ pv,
                                                     float* __restrict__ part, int R) {
    extern __shared__ float sm[];
    const int r = blockIdx.x, h = blockIdx.y, pos = t.row_pos[r];
    int lo, nb;
    sattn_range(b, pos, lo, nb);
    const int total = nb + pos - lo + 1;
    const int per = ((total + (int)gridDim.z - 1) / (int)gridDim.z + 127) / 128 * 128;
    const int n_lo = blockIdx.z * per, n_hi = min(total, n_lo + per);
    float m = -INFINITY, l = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (n_lo < n_hi) sattn_sweep<OT>(t, b, P, ldp, kc, vc, pk, pv, sm, r, h, n_lo, n_hi, lo, nb, m, l, acc);
    float* o = part + (((size_t)blockIdx.z * R + r) * (b.heads * sa_maps(b)) + h) * (b.vdim + 2);
    if (threadIdx.x == 0) { o[0] = m; o[1] = l; }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
        const int c = threadIdx.x + cc * blockDim.x;
        if (c < b.vdim) o[2 + c] = acc[cc];
    }
}
template <typename OT>
__global__ void __launch_bounds__(128) k_sattn_join(SoftAttn b, const float* __restrict__ P, int ldp, const float* __restrict__ part, int R, int splits,
                                                    OT* __restrict__ out, int ld_out) {
    // splits <= 32: one warp fetches every split's maximum and denominator at once and turns them into the splits' weights; the value sums
    // are then folded in order without waiting on a load per split
    __shared__ float sw[32];
    __shared__ float s_inv;
    const int r = blockIdx.x, h = blockIdx.y;
    const size_t stride = (size_t)R * (b.heads * sa_maps(b)) * (b.vdim + 2);
    const float* p0 = part + ((size_t)r * (b.heads * sa_maps(b)) + h) * (b.vdim + 2);
    if (threadIdx.x < 32) {
        const int k = threadIdx.x;
        const float mk = k < splits ? p0[k * stride] : -INFINITY, lk = k < splits ? p0[k * stride + 1] : 0.0f;
        const float sink = b.sink ? b.sink[h / sa_maps(b)] : -INFINITY;
        const float M = fmaxf(sink, warp_max(mk));
        const float w = mk == -INFINITY ? 0.0f : expf(mk - M);
        float l = warp_sum(lk * w);
        if (b.sink) l += expf(sink - M);
        sw[k] = w;
        if (k == 0) s_inv = 1.0f / l;
    }
    __syncthreads();
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // eight splits at a time: all their loads are issued before the first multiply-add waits on one (sw is 0 beyond `splits`)
    for (int k0 = 0; k0 < splits; k0 += 8) {
        float v[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const bool on = sw[k0 + i] != 0.0f;          // an empty key range left its value sums unwritten
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const int c = threadIdx.x + cc * blockDim.x;
                v[i][cc] = (on && c < b.vdim) ? p0[(size_t)(k0 + i) * stride + 2 + c] : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int cc = 0; cc < 4; cc++) acc[cc] = fmaf(v[i][cc], sw[k0 + i], acc[cc]);
    }
    sattn_store<OT>(b, P, ldp, r, h, s_inv, acc, out, ld_out);
}

// ------------------------------------------------------------------------------------------------ PolyNorm
// act = a N(z) + b N(z^2) + c N(z^3) + e, N(v) = v / sqrt(mean(v^2) + eps) over the row's ff values; coef = (a, b, c, e)
template <typename OT>
__global__ void __launch_bounds__(256) k_polynorm(const float* __restrict__ G, int ldg, int ff, float eps, const float* __restrict__ coef,
                                                  OT* __restrict__ out, int ld_out) {
    __shared__ float red[3][9];
    const int r = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const float* z = G + (size_t)r * ldg;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    constexpr int KEEP = 8;
    const bool keep = ff % 4 == 0 && ldg % 4 == 0 && ld_out % 4 == 0 && ff <= 4 * KEEP * (int)blockDim.x;     // the row stays in registers: read once
    float4 vz[KEEP];
    if (keep) {
#pragma unroll
        for (int i = 0; i < KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < ff) {
                const float4 v = *reinterpret_cast<const float4*>(z + c);
                vz[i] = v;
                const float a = v.x * v.x, b = v.y * v.y, cc = v.z * v.z, d = v.w * v.w;
                s2 += a + b + cc + d; s4 += a * a + b * b + cc * cc + d * d; s6 += a * a * a + b * b * b + cc * cc * cc + d * d * d;
            }
        }
    } else {
        for (int c = threadIdx.x; c < ff; c += blockDim.x) { const float v = z[c], v2 = v * v; s2 += v2; s4 += v2 * v2; s6 += v2 * v2 * v2; }
    }
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);         // the three sums share one pass and one barrier
    if (lane == 0) { red[0][wid] = s2; red[1][wid] = s4; red[2][wid] = s6; }
    __syncthreads();
    s2 = s4 = s6 = 0.0f;
    for (int w = 0; w < 8; w++) { s2 += red[0][w]; s4 += red[1][w]; s6 += red[2][w]; }
    const float n = (float)ff;
    const float k1 = coef[0] / sqrtf(s2 / n + eps), k2 = coef[1] / sqrtf(s4 / n + eps), k3 = coef[2] / sqrtf(s6 / n + eps), k0 = coef[3];
    if (keep) {
#pragma unroll
        for (int i = 0; i < KEEP; i++) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < ff) {
                const float4 v = vz[i];
                store4(out + (size_t)r * ld_out + c, fmaf(v.x, fmaf(v.x, fmaf(v.x, k3, k2), k1), k0), fmaf(v.y, fmaf(v.y, fmaf(v.y, k3, k2), k1), k0),
                       fmaf(v.z, fmaf(v.z, fmaf(v.z, k3, k2), k1), k0), fmaf(v.w, fmaf(v.w, fmaf(v.w, k3, k2), k1), k0));
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < ff; c += blockDim.x) {
        const float v = z[c];
        out[(size_t)r * ld_out + c] = cvt<OT>(fmaf(v, fmaf(v, fmaf(v, k3, k2), k1), k0));
    }
}

// ------------------------------------------------------------------------------------------------ routed experts
// lane-partial dot of an operand row with a bf16 weight row over K (a multiple of 64; both rows 16-byte aligned)
template <typename OT>
__device__ __forceinline__ float lane_dot(const OT* __restrict__ a, const bf16* __restrict__ w, int K, int lane) {
    float s = 0.0f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + k));
        float av[8];
        load8<OT>(a + k, av);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s = fmaf(av[2 * i], __uint_as_float(ww[i] << 16), s);
            s = fmaf(av[2 * i + 1], __uint_as_float(ww[i] & 0xffff0000u), s);
        }
    }
    return s;
}
// Few rows: pair (row r, choice k) with expert e streams that expert's up matrix once: act[pair][c] = w * relu(up_e[c] . x_r)^2 for
// c < ff, zero up to the padded width kfp.  Pairs that chose an identity expert write nothing (their rows of act are not read).
// grid (R * top, column groups); a warp takes one column at a time.  w_up [n_experts * ff][ldw].
template <typename OT>
__global__ void __launch_bounds__(256) k_moe_up_rows(const OT* __restrict__ X, int ldx, int K, const bf16* __restrict__ w_up, int ldw, int ff, int kfp,
                                                     int n_experts, int top, const int* __restrict__ sel_idx, const float* __restrict__ sel_w,
                                                     OT* __restrict__ act) {
    const int pair = blockIdx.x, r = pair / top, e = sel_idx[pair];
    if (e >= n_experts) return;
    const float wt = sel_w[pair];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const OT* x = X + (size_t)r * ldx;
    for (int c = blockIdx.y * nw + warp; c < kfp; c += gridDim.y * nw) {
        float u = 0.0f;
        if (c < ff) u = warp_sum(lane_dot<OT>(x, w_up + ((size_t)e * ff + c) * ldw, K, lane));
        if (lane == 0) { const float a = fmaxf(u, 0.0f); act[(size_t)pair * kfp + c] = cvt<OT>(wt * a * a); }
    }
}
// Y[r][c] = sum over the row's expert choices of down_e[c] . act[pair]; w_down [n_experts][width][kfp].  grid (R, column groups).
template <typename OT>
__global__ void __launch_bounds__(256) k_moe_down_rows(const OT* __restrict__ act, int kfp, const bf16* __restrict__ w_down, int width, int n_experts, int top,
                                                       const int* __restrict__ sel_idx, float* __restrict__ Y, int ldy) {
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int c = blockIdx.y * nw + warp; c < width; c += gridDim.y * nw) {
        float y = 0.0f;
        for (int k = 0; k < top; k++) {
            const int e = sel_idx[(size_t)r * top + k];
            if (e >= n_experts) continue;
            y += lane_dot<OT>(act + ((size_t)r * top + k) * kfp, w_down + ((size_t)e * width + c) * kfp, kfp, lane);
        }
        y = warp_sum(y);
        if (lane == 0) Y[(size_t)r * ldy + c] = y;
    }
}

}  // namespace seq
}  // namespace gtb
