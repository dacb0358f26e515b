// gtb_seq_mixers_tiled.cuh -- tiled kernels of the post-norm layer style for prompt portions in bf16 mode:
//   * k_sattn_mma: windowed softmax attention with pooled blocks and a sink on mma.sync m16n8k16 (the softmax sibling of k_sigattn_mma)
//   * k_moe_group / k_moe_gather: rows sorted by chosen expert into 128-row-aligned groups for the grouped tensor-core products
#pragma once
#include "gtb_seq_mixers.cuh"

namespace gtb {
namespace seq {

__device__ __forceinline__ float sa_tanh(float z) {
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(z));
    return th;
}

// A CTA owns 64 consecutive rows of one segment and one query head (4 warps x 16 rows).  It sweeps, in tiles of 64 keys, first the
// pooled blocks that its last row sees (fp32 means converted to bf16 on the way into shared memory), then the tokens from the first
// row's window start to the last row: S = Q K^T, score = cap(scale S) under the row's own mask (block b: (b + 1) pool <= pos - window + 1;
// token j: pos - window < j <= pos), online softmax in fp32 whose running maximum starts at the sink (so the sink's term is
// exp(sink - max) at the end and counts once), O += P V with P as bf16 A fragments straight from the accumulator registers.
// Soft-capping uses the special-function tanh (relative error 2^-11, below the bf16 rounding of the weights that follow).
template <int DP, int VP>
__global__ void __launch_bounds__(128) k_sattn_mma(PassTables t, SoftAttn b, int S, const float* __restrict__ P, int ldp, const bf16* __restrict__ kc,
                                                   const bf16* __restrict__ vc, const float* __restrict__ pk, const float* __restrict__ pv,
                                                   bf16* __restrict__ out, int ld_out, float* __restrict__ out_f, int ld_f) {
    constexpr int LQ = DP + 8, LV = VP + 8;
    extern __shared__ __align__(16) unsigned char sa_raw[];
    bf16* sq = reinterpret_cast<bf16*>(sa_raw);          // [64][LQ]
    bf16* sk0 = sq + 64 * LQ;                           // [2][64][LQ]: key tiles, double-buffered
    bf16* sv0 = sk0 + 2 * 64 * LQ;                      // [2][64][LV]
    int seg, q0;
    if (!sa_find_tile(t, S, blockIdx.x, seg, q0)) return;
    const int M = sa_maps(b), h = blockIdx.y, hd = h / M, g = hd / (b.heads / b.kv_heads), ku = g * M + h % M;     // h: query unit
    const int slot = t.seg_slot[seg], row0 = t.seg_row0[seg] + q0, nq = min(64, t.seg_len[seg] - q0);
    const int pos0 = t.row_pos[row0];                    // position of the tile's first row; row i sits at pos0 + i
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    for (int e = threadIdx.x; e < 64 * DP; e += 128) {
        const int r = e / DP, i = e % DP;
        sq[r * LQ + i] = __float2bfloat16_rn((r < nq && i < b.dim) ? P[(size_t)(row0 + r) * ldp + b.q_off + h * b.dim + i] : 0.0f);
    }
    const size_t kld = (size_t)b.kv_heads * M * b.dim, vld = (size_t)b.kv_heads * b.vdim;
    const bf16* kbase = kc + (size_t)slot * b.max_ctx * kld + (size_t)ku * b.dim;
    const bf16* vbase = vc + (size_t)slot * b.max_ctx * vld + (size_t)g * b.vdim;
    const float* pkb = pk ? pk + (size_t)slot * b.max_blocks * kld + (size_t)ku * b.dim : nullptr;
    const float* pvb = pv ? pv + (size_t)slot * b.max_blocks * vld + (size_t)g * b.vdim : nullptr;
    const bool vec = (b.dim % 8 == 0) && (b.vdim % 8 == 0);
    const int last = pos0 + nq - 1;                      // last position of the tile
    int t_lo, nb_tile;
    sattn_range(b, last, t_lo, nb_tile);                 // blocks the last row sees: the most of any row
    { int nb0; sattn_range(b, pos0, t_lo, nb0); }     // the first row's first token: the lowest of any row
    const int n_bt = (nb_tile + 63) / 64, n_it = n_bt + (last - t_lo) / 64 + 1;
    const uint32_t sq_a = (uint32_t)__cvta_generic_to_shared(sq);
    auto load_tile = [&](int st, int it) {
        bf16* sk = sk0 + st * 64 * LQ;
        bf16* sv = sv0 + st * 64 * LV;
        if (it < n_bt) {
            const int b0 = it * 64, nk = min(64, nb_tile - b0);
            for (int e = threadIdx.x; e < 64 * DP; e += 128) {
                const int r = e / DP, i = e % DP;
                sk[r * LQ + i] = __float2bfloat16_rn((r < nk && i < b.dim) ? pkb[(size_t)(b0 + r) * kld + i] : 0.0f);
            }
            for (int e = threadIdx.x; e < 64 * VP; e += 128) {
                const int r = e / VP, i = e % VP;
                sv[r * LV + i] = __float2bfloat16_rn((r < nk && i < b.vdim) ? pvb[(size_t)(b0 + r) * vld + i] : 0.0f);
            }
        } else {
            const int j0 = t_lo + (it - n_bt) * 64, nk = min(64, last + 1 - j0);
            if (vec) {
                const uint32_t ka = (uint32_t)__cvta_generic_to_shared(sk), va = (uint32_t)__cvta_generic_to_shared(sv);
                for (int e = threadIdx.x; e < 64 * (DP / 8); e += 128) {
                    const int r = e / (DP / 8), c8 = (e % (DP / 8)) * 8;
                    const bool ok = r < nk && c8 < b.dim;
                    sa_cp16(ka + (uint32_t)((r * LQ + c8) * 2), ok ? (const void*)(kbase + (size_t)(j0 + r) * kld + c8) : (const void*)kbase, ok);
                }
                for (int e = threadIdx.x; e < 64 * (VP / 8); e += 128) {
                    const int r = e / (VP / 8), c8 = (e % (VP / 8)) * 8;
                    const bool ok = r < nk && c8 < b.vdim;
                    sa_cp16(va + (uint32_t)((r * LV + c8) * 2), ok ? (const void*)(vbase + (size_t)(j0 + r) * vld + c8) : (const void*)vbase, ok);
                }
            } else {
                for (int e = threadIdx.x; e < 64 * DP; e += 128) {
                    const int r = e / DP, i = e % DP;
                    sk[r * LQ + i] = (r < nk && i < b.dim) ? kbase[(size_t)(j0 + r) * kld + i] : __float2bfloat16_rn(0.0f);
                }
                for (int e = threadIdx.x; e < 64 * VP; e += 128) {
                    const int r = e / VP, i = e % VP;
                    sv[r * LV + i] = (r < nk && i < b.vdim) ? vbase[(size_t)(j0 + r) * vld + i] : __float2bfloat16_rn(0.0f);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // this thread's two rows: positions, first visible token, number of visible blocks
    const int p_lo = pos0 + warp * 16 + gq, p_hi = p_lo + 8;
    int tl_lo, tl_hi, nb_lo, nb_hi;
    sattn_range(b, p_lo, tl_lo, nb_lo);
    sattn_range(b, p_hi, tl_hi, nb_hi);
    const int pw0 = pos0 + warp * 16, pw1 = pw0 + 15;      // the warp's rows
    int wl_dummy, nb_w, wl0, nb_w0;
    sattn_range(b, pw1, wl_dummy, nb_w);
    sattn_range(b, pw0, wl0, nb_w0);                      // first token the warp's first row sees: no row of the warp sees an earlier one
    const float sink = b.sink ? b.sink[hd] : -INFINITY;
    float m_lo = sink, m_hi = sink, l_lo = 0.0f, l_hi = 0.0f;
    float o[VP / 8][4];
#pragma unroll
    for (int n = 0; n < VP / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    const float inv_cap = b.softcap > 0.0f ? 1.0f / b.softcap : 0.0f;
    load_tile(0, 0);
    for (int it = 0; it < n_it; it++) {
        const int st = it & 1;
        const bool more = it + 1 < n_it;
        if (more) load_tile(st ^ 1, it + 1);             // its previous reader passed the barrier at the end of the last iteration
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const bool is_blk = it < n_bt;
        const int k0 = is_blk ? it * 64 : t_lo + (it - n_bt) * 64;
        const bool skip = is_blk ? (k0 >= nb_w) : (k0 > pw1 || k0 + 63 < wl0);
        if (skip) { __syncthreads(); continue; }        // no row of this warp sees a key of the tile
        const uint32_t sk_a = (uint32_t)__cvta_generic_to_shared(sk0 + st * 64 * LQ), sv_a = (uint32_t)__cvta_generic_to_shared(sv0 + st * 64 * LV);
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < DP / 16; kk++) {
            uint32_t a[4];
            sa_ldsm_x4(sq_a + (uint32_t)(((warp * 16 + (lane & 15)) * LQ + kk * 16 + (lane >> 4) * 8) * 2), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int n2 = 0; n2 < 4; n2++) {
                uint32_t b0, b1, b2, b3;
                sa_ldsm_x4(sk_a + (uint32_t)(((n2 * 16 + (lane & 7) + (lane >> 4) * 8) * LQ + kk * 16 + ((lane >> 3) & 1) * 8) * 2), b0, b1, b2, b3);
                sa_mma(sc[2 * n2], a, b0, b1);
                sa_mma(sc[2 * n2 + 1], a, b2, b3);
            }
        }
        // scores under each row's mask; rows gq and gq + 8 of the warp's 16, keys k0 + 8 n + 2 tq (+1)
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; n++) {
#pragma unroll
            for (int x = 0; x < 4; x++) {
                const int key = k0 + n * 8 + tq * 2 + (x & 1);
                const bool hi = x >= 2;
                const bool vis = is_blk ? key < (hi ? nb_hi : nb_lo) : (key <= (hi ? p_hi : p_lo) && key >= (hi ? tl_hi : tl_lo));
                float s = sc[n][x] * b.scale;
                if (b.softcap > 0.0f) s = b.softcap * sa_tanh(s * inv_cap);
                s = vis ? s : -INFINITY;
                sc[n][x] = s;
                if (hi) mx_hi = fmaxf(mx_hi, s); else mx_lo = fmaxf(mx_lo, s);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float c_lo = m_lo == -INFINITY ? 0.0f : __expf(m_lo - mn_lo), c_hi = m_hi == -INFINITY ? 0.0f : __expf(m_hi - mn_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        l_lo *= c_lo; l_hi *= c_hi;
#pragma unroll
        for (int n = 0; n < VP / 8; n++) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
        uint32_t w[8][2];
#pragma unroll
        for (int n = 0; n < 8; n++) {
            const float w0 = sc[n][0] == -INFINITY ? 0.0f : __expf(sc[n][0] - mn_lo), w1 = sc[n][1] == -INFINITY ? 0.0f : __expf(sc[n][1] - mn_lo);
            const float w2 = sc[n][2] == -INFINITY ? 0.0f : __expf(sc[n][2] - mn_hi), w3 = sc[n][3] == -INFINITY ? 0.0f : __expf(sc[n][3] - mn_hi);
            l_lo += w0 + w1; l_hi += w2 + w3;
            w[n][0] = sa_pack(w0, w1);
            w[n][1] = sa_pack(w2, w3);
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {                 // 16 keys per step
            const uint32_t a[4] = {w[2 * kk][0], w[2 * kk][1], w[2 * kk + 1][0], w[2 * kk + 1][1]};
#pragma unroll
            for (int n2 = 0; n2 < VP / 16; n2++) {
                uint32_t b0, b1, b2, b3;
                sa_ldsm_x4_t(sv_a + (uint32_t)(((kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LV + n2 * 16 + (lane >> 4) * 8) * 2), b0, b1, b2, b3);
                sa_mma(o[2 * n2], a, b0, b1);
                sa_mma(o[2 * n2 + 1], a, b2, b3);
            }
        }
        __syncthreads();                                 // this stage may be refilled from the next iteration on
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (b.sink) { l_lo += __expf(sink - m_lo); l_hi += __expf(sink - m_hi); }
    const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
    const int r_lo = warp * 16 + gq, r_hi = r_lo + 8;
    if (out_f) {                                         // fp32, no gate and no weight: a later kernel combines the query units
#pragma unroll
        for (int n = 0; n < VP / 8; n++) {
            const int c = n * 8 + tq * 2;
#pragma unroll
            for (int x = 0; x < 2; x++) {
                if (c + x >= b.vdim) continue;
                if (r_lo < nq) out_f[(size_t)(row0 + r_lo) * ld_f + h * b.vdim + c + x] = o[n][x] * i_lo;
                if (r_hi < nq) out_f[(size_t)(row0 + r_hi) * ld_f + h * b.vdim + c + x] = o[n][2 + x] * i_hi;
            }
        }
        return;
    }
    const float os = b.out_scale != 0.0f ? b.out_scale : 1.0f;
#pragma unroll
    for (int n = 0; n < VP / 8; n++) {
        const int c = n * 8 + tq * 2;
#pragma unroll
        for (int x = 0; x < 2; x++) {
            if (c + x >= b.vdim) continue;
            if (r_lo < nq) {
                float v = o[n][x] * i_lo * os;
                if (b.gate) { const float gt = P[(size_t)(row0 + r_lo) * ldp + b.g_off + (b.gate == 3 ? hd : h * b.vdim + c + x)]; v *= b.gate >= 2 ? sigmoidf_(gt) : gt * sigmoidf_(gt); }
                out[(size_t)(row0 + r_lo) * ld_out + b.a_off + h * b.vdim + c + x] = __float2bfloat16_rn(v);
            }
            if (r_hi < nq) {
                float v = o[n][2 + x] * i_hi * os;
                if (b.gate) { const float gt = P[(size_t)(row0 + r_hi) * ldp + b.g_off + (b.gate == 3 ? hd : h * b.vdim + c + x)]; v *= b.gate >= 2 ? sigmoidf_(gt) : gt * sigmoidf_(gt); }
                out[(size_t)(row0 + r_hi) * ld_out + b.a_off + h * b.vdim + c + x] = __float2bfloat16_rn(v);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ rows grouped by expert
// One CTA.  Counts the (row, choice) pairs of every expert, lays the experts' groups out one after the other with every group starting
// on a multiple of 128 rows (one M tile of the tensor-core product never mixes experts), gives every pair its row in that layout
// (dst; -1 for an identity expert) and every M tile its expert (tile_e; -1 beyond the last group).  Shared memory: 2 n_experts ints.
__global__ void __launch_bounds__(1024) k_moe_group(const int* __restrict__ sel_idx, int n_pairs, int n_experts, int* __restrict__ dst,
                                                    int* __restrict__ tile_e, int n_tiles) {
    extern __shared__ int sg[];
    int* cnt = sg;                  // [n_experts] pairs per expert, then the running fill of the group
    int* start = sg + n_experts;    // [n_experts] first row of the group
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) { const int e = sel_idx[p]; if (e < n_experts) atomicAdd(&cnt[e], 1); }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_experts; e++) {
            start[e] = at;
            const int nt = (cnt[e] + 127) / 128;
            for (int k = 0; k < nt; k++) tile_e[at / 128 + k] = e;
            at += nt * 128;
            cnt[e] = 0;
        }
        for (int k = at / 128; k < n_tiles; k++) tile_e[k] = -1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = sel_idx[p];
        dst[p] = e < n_experts ? start[e] + atomicAdd(&cnt[e], 1) : -1;
    }
}
// Xg[dst[pair]] = X[pair / top] (bf16 rows of ld elements, 16-byte pieces); rw[dst[pair]] = the pair's weight
__global__ void __launch_bounds__(128) k_moe_gather(const bf16* __restrict__ X, int ld, int top, const int* __restrict__ dst, const float* __restrict__ sel_w,
                                                    bf16* __restrict__ Xg, float* __restrict__ rw) {
    const int pair = blockIdx.x, d = dst[pair];
    if (d < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(X + (size_t)(pair / top) * ld);
    uint4* out = reinterpret_cast<uint4*>(Xg + (size_t)d * ld);
    for (int i = threadIdx.x; i < ld / 8; i += blockDim.x) out[i] = src[i];
    if (threadIdx.x == 0) rw[d] = sel_w[pair];
}

}  // namespace seq
}  // namespace gtb
