// A short causal convolution over time on every channel of the projected q, k and v, fused with the rotary
// encoding of q and k and the append of k and v to the paged cache.
//
//   y[p, c] = sum_{j < taps} w[j, c] * u[p - taps + 1 + j, c],   u = 0 before the sequence's start (w tap-major: [taps, channels]),
//
// u being the projections [T, nh*hd | nkv*hd | nkv*hdv] of the step's tokens (float).  Values of u at
// positions before the step's first token come from the sequence's ring: ring[slot][p % taps][c] holds u[p, c]
// for the last `taps` positions the sequence has been given.  Because a position always lands in the same
// place of the ring, a step that is run again for the same position (a decode step launched ahead and then
// dropped) overwrites what its first run left, and nothing needs to be rolled back.  The ring is written by a
// second kernel after the first has read it (the places written and read overlap modulo taps).
//
// Then, as in the plain rope_append kernel: the first `rot` dimensions of every q and k head are rotated by
// angle = float(pos) * inv_freq[i] (pairing 0: (i, i + rot/2); pairing 1: (2i, 2i + 1)), q goes to q_out, k and v
// into the token's place in the pages.  Value heads may have a size of their own (hdv).  All arithmetic is float,
// with the products of the convolution added in ascending j.
#include "common.cuh"

namespace {

struct ConvArgs {
    const float* qkv; const float* conv_w; const float* ring; const int* slots; const int* cu_seqlens;
    const int* token_seq; const int* token_pos; const int* table; const float* inv_freq;
    int table_stride, nh, nkv, hd, hdv, rot, pairing, taps, page_size, n_pages, write_cache, heads_per_block, ctot;
};

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
conv_rope_append_kernel(ConvArgs a, TQ* __restrict__ q_out, TC* __restrict__ k_pages, TC* __restrict__ v_pages, int* status) {
    extern __shared__ __align__(16) float cs[];    // [rot/2] cos, then [rot/2] sin of this token's angles
    ik_pdl_wait();
    IK_AFTER_WAIT(a.qkv);
    IK_AFTER_WAIT(a.ring);
    IK_AFTER_WAIT(a.slots);
    IK_AFTER_WAIT(a.cu_seqlens);
    IK_AFTER_WAIT(a.token_seq);
    IK_AFTER_WAIT(a.token_pos);
    IK_AFTER_WAIT(a.table);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, half = a.rot / 2, tid = threadIdx.y * blockDim.x + threadIdx.x;
    const int nh = a.nh, nkv = a.nkv, hd = a.hd, hdv = a.hdv, taps = a.taps, ctot = a.ctot;
    const int head_lo = blockIdx.y * a.heads_per_block;
    const int head_hi = min(head_lo + a.heads_per_block, nh + 2 * nkv);
    const int pos = a.token_pos[t], seq = a.token_seq[t];
    const int first = a.cu_seqlens[seq];                 // the sequence's first token of this step
    const int pos_start = pos - (t - first);             // ... and its position
    const float* ring = a.ring ? a.ring + (size_t)a.slots[seq] * taps * ctot : nullptr;
    if (head_lo < nh + nkv) {
        for (int i = tid; i < half; i += blockDim.x * blockDim.y) {
            const float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            cs[i] = cosf(ang);
            cs[half + i] = sinf(ang);
        }
    }
    size_t page_row = 0;
    bool page_ok = false;
    if (a.write_cache && head_hi > nh) {
        const int page = a.table[(size_t)seq * a.table_stride + pos / a.page_size];
        page_ok = page >= 0 && page < a.n_pages;
        if (!page_ok) { if (tid == 0) ik_set_status(status, IK_STATUS_WRITE_NO_PAGE); }
        else page_row = (size_t)page * nkv * a.page_size + (pos % a.page_size);
    }
    __syncthreads();
    auto conv_at = [&](int c) -> float {
        const float* here = a.qkv + (size_t)t * ctot + c;
        if (taps <= 0) return *here;
        float acc = 0.f;
        for (int j = 0; j < taps; j++) {
            const int back = taps - 1 - j, p = pos - back;
            if (p < 0) continue;
            const float u = p >= pos_start ? *(here - (size_t)back * ctot) : ring[(size_t)(p % taps) * ctot + c];
            acc = fmaf(a.conv_w[(size_t)j * ctot + c], u, acc);
        }
        return acc;
    };
    for (int head = head_lo + threadIdx.y; head < head_hi; head += blockDim.y) {
        if (head < nh + nkv) {
            const bool is_q = head < nh;
            if (!is_q && !page_ok) continue;
            const int c0 = head * hd;                                            // q heads, then k heads: all of size hd
            TQ* qdst = q_out + ((size_t)t * nh + head) * hd;
            TC* kdst = k_pages + (page_row + (size_t)(head - nh) * a.page_size) * hd;
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const int i0 = a.pairing == 0 ? i : 2 * i, i1 = a.pairing == 0 ? i + half : 2 * i + 1;
                const float c = cs[i], sn = cs[half + i];
                const float x0 = conv_at(c0 + i0), x1 = conv_at(c0 + i1);
                const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
                const float r1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sn));
                if (is_q) { ik_st(qdst, i0, r0); ik_st(qdst, i1, r1); }
                else { ik_st(kdst, i0, r0); ik_st(kdst, i1, r1); }
            }
            for (int i = a.rot + threadIdx.x; i < hd; i += blockDim.x) {
                const float v = conv_at(c0 + i);
                if (is_q) ik_st(qdst, i, v);
                else ik_st(kdst, i, v);
            }
        } else if (page_ok) {
            const int g = head - nh - nkv;
            const int c0 = (nh + nkv) * hd + g * hdv;
            TC* vdst = v_pages + (page_row + (size_t)g * a.page_size) * hdv;
            for (int i = threadIdx.x; i < hdv; i += blockDim.x) ik_st(vdst, i, conv_at(c0 + i));
        }
    }
}

// The same, four neighbouring channels a thread with 16-byte loads and stores: for neighbouring rotary pairs (pairing 1) or
// no rotation, and head sizes, rotated width and channel count that are multiples of 4.  A block takes 1024 channels of
// one token.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
conv_rope_append_vec_kernel(ConvArgs a, TQ* __restrict__ q_out, TC* __restrict__ k_pages, TC* __restrict__ v_pages, int* status) {
    extern __shared__ __align__(16) float cs[];    // [rot/2] cos, then [rot/2] sin of this token's angles
    ik_pdl_wait();
    IK_AFTER_WAIT(a.qkv);
    IK_AFTER_WAIT(a.ring);
    IK_AFTER_WAIT(a.slots);
    IK_AFTER_WAIT(a.cu_seqlens);
    IK_AFTER_WAIT(a.token_seq);
    IK_AFTER_WAIT(a.token_pos);
    IK_AFTER_WAIT(a.table);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, half = a.rot / 2;
    const int nh = a.nh, nkv = a.nkv, hd = a.hd, hdv = a.hdv, taps = a.taps, ctot = a.ctot;
    const int pos = a.token_pos[t], seq = a.token_seq[t];
    const int pos_start = pos - (t - a.cu_seqlens[seq]);
    const int c_lo = blockIdx.y * 1024;
    const int q_end = nh * hd, k_end = (nh + nkv) * hd;
    if (c_lo < k_end) {
        for (int i = threadIdx.x; i < half; i += 256) {
            const float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            cs[i] = cosf(ang);
            cs[half + i] = sinf(ang);
        }
    }
    __syncthreads();
    const int c = c_lo + 4 * threadIdx.x;
    if (c >= ctot) return;
    const float* ring = a.ring ? a.ring + (size_t)a.slots[seq] * taps * ctot : nullptr;
    const float* here = a.qkv + (size_t)t * ctot + c;
    float4 y;
    if (taps <= 0) {
        y = *reinterpret_cast<const float4*>(here);
    } else {
        y = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < taps; j++) {
            const int back = taps - 1 - j, p = pos - back;
            if (p < 0) continue;
            const float4 u = *reinterpret_cast<const float4*>(p >= pos_start ? here - (size_t)back * ctot : ring + (size_t)(p % taps) * ctot + c);
            const float4 w = *reinterpret_cast<const float4*>(a.conv_w + (size_t)j * ctot + c);
            y.x = fmaf(w.x, u.x, y.x); y.y = fmaf(w.y, u.y, y.y); y.z = fmaf(w.z, u.z, y.z); y.w = fmaf(w.w, u.w, y.w);
        }
    }
    if (c < k_end) {
        const int i = c % hd;                                   // q and k heads have the same size
        if (i < a.rot) {
            const float c0 = cs[i / 2], s0 = cs[half + i / 2], c1 = cs[i / 2 + 1], s1 = cs[half + i / 2 + 1];
            const float4 r = make_float4(__fsub_rn(__fmul_rn(y.x, c0), __fmul_rn(y.y, s0)), __fadd_rn(__fmul_rn(y.y, c0), __fmul_rn(y.x, s0)),
                                         __fsub_rn(__fmul_rn(y.z, c1), __fmul_rn(y.w, s1)), __fadd_rn(__fmul_rn(y.w, c1), __fmul_rn(y.z, s1)));
            y = r;
        }
        if (c < q_end) { ik_st4(q_out, (size_t)t * q_end + c, y); return; }
    }
    if (!a.write_cache) return;
    const int page = a.table[(size_t)seq * a.table_stride + pos / a.page_size];
    if (page < 0 || page >= a.n_pages) { ik_set_status(status, IK_STATUS_WRITE_NO_PAGE); return; }
    const size_t page_row = (size_t)page * nkv * a.page_size + (pos % a.page_size);
    if (c < k_end) {
        const int g = (c - q_end) / hd, i = (c - q_end) % hd;
        ik_st4(k_pages, (page_row + (size_t)g * a.page_size) * hd + i, y);
    } else {
        const int g = (c - k_end) / hdv, i = (c - k_end) % hdv;
        ik_st4(v_pages, (page_row + (size_t)g * a.page_size) * hdv + i, y);
    }
}

// ring[slot][p % taps][:] = u[p, :] for the last min(taps, new) positions of every sequence of the step
__global__ void conv_ring_write_kernel(const float* __restrict__ qkv, float* __restrict__ ring, const int* __restrict__ slots,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens, int taps, int ctot) {
    ik_pdl_wait();
    IK_AFTER_WAIT(qkv);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x;
    const int first = cu_seqlens[b], n_new = cu_seqlens[b + 1] - first, end = kv_lens[b], pos_start = end - n_new;
    float* mine = ring + (size_t)slots[b] * taps * ctot;
    for (int p = max(pos_start, end - taps); p < end; p++) {
        const float* src = qkv + (size_t)(first + p - pos_start) * ctot;
        float* dst = mine + (size_t)(p % taps) * ctot;
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ctot; c += gridDim.y * blockDim.x) dst[c] = src[c];
    }
}

}  // namespace

IK_EXPORT int ik_conv_rope_append(const float* qkv, const float* conv_w, float* ring, const int* slots, const int* cu_seqlens,
                                  const int* kv_lens, void* q_out, int q_dtype, void* k_pages, void* v_pages, int cache_dtype,
                                  const int* token_seq, const int* token_pos, const int* table, int table_stride,
                                  const float* inv_freq, int T, int n_seqs, int nh, int nkv, int hd, int hdv, int rot, int pairing,
                                  int taps, int page_size, int n_pages, int write_cache, int* status, cudaStream_t stream) {
    if (T < 0 || n_seqs < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || hdv <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0 || taps < 0)
        return IK_BAD_ARGUMENT;
    if ((rot > 0 && !inv_freq) || (taps > 0 && !conv_w) || (taps > 1 && !ring)) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const int hpb = T >= 256 ? 16 : 4;
    ConvArgs a = {qkv, conv_w, ring, slots, cu_seqlens, token_seq, token_pos, table, inv_freq, table_stride, nh, nkv, hd, hdv,
                  rot, pairing, taps, page_size, n_pages, write_cache, hpb, (nh + nkv) * hd + nkv * hdv};
    dim3 grid(T, (nh + 2 * nkv + hpb - 1) / hpb);
    const dim3 threads(32, 8);
    const size_t smem = (size_t)rot * sizeof(float);
    const bool vec = (rot == 0 || pairing == 1) && hd % 4 == 0 && hdv % 4 == 0 && rot % 4 == 0 && ((uintptr_t)qkv % 16) == 0 &&
                     ((uintptr_t)conv_w % 16) == 0 && ((uintptr_t)ring % 16) == 0 && ((uintptr_t)q_out % 16) == 0 &&
                     ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0;
    const dim3 vgrid(T, (a.ctot + 1023) / 1024);
#define IK_CONV(TQ, TC)                                                                                                                \
    if (vec) IK_RETURN_IF_ERROR(ik_launch(conv_rope_append_vec_kernel<TQ, TC>, vgrid, 256, smem, stream, a, (TQ*)q_out, (TC*)k_pages, (TC*)v_pages, status)); \
    else IK_RETURN_IF_ERROR(ik_launch(conv_rope_append_kernel<TQ, TC>, grid, threads, smem, stream, a, (TQ*)q_out, (TC*)k_pages, (TC*)v_pages, status))
    if (q_dtype == IK_F32 && cache_dtype == IK_F32) { IK_CONV(float, float); }
    else if (q_dtype == IK_BF16 && cache_dtype == IK_BF16) { IK_CONV(__nv_bfloat16, __nv_bfloat16); }
    else if (q_dtype == IK_F32 && cache_dtype == IK_BF16) { IK_CONV(float, __nv_bfloat16); }
    else if (q_dtype == IK_BF16 && cache_dtype == IK_F32) { IK_CONV(__nv_bfloat16, float); }
    else return IK_BAD_ARGUMENT;
#undef IK_CONV
    if (taps > 1 && write_cache && n_seqs > 0) {
        const int per = (a.ctot + 255) / 256;
        dim3 g2(n_seqs, per < 16 ? per : 16);
        IK_RETURN_IF_ERROR(ik_launch(conv_ring_write_kernel, g2, 256, 0, stream, qkv, ring, slots, cu_seqlens, kv_lens, taps, a.ctot));
    }
    IK_LAUNCH_STATUS();
}
