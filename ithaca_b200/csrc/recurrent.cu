// Mixers that carry a state of fixed size from token to token: a short causal convolution with bias and
// activation, the selective scan, and linear attention with a constant decay per head.
//
// All of them work on the step's token-major batch: sequence b brings tokens cu_seqlens[b] .. cu_seqlens[b+1] - 1,
// which sit at positions kv_lens[b] - n_b .. kv_lens[b] - 1; its state lives in slot slots[b].  A sequence whose
// first token sits at position 0 starts from zeros whatever its slot holds.
//
// State that a step replaces (the scan's and the linear attention's) is kept twice, by the parity of the
// position it belongs to: a step that ends at position e reads the copy of parity (first - 1) & 1 and writes
// the copy of parity e & 1.  A decode step therefore never overwrites what it read, so running the same step
// again (a captured graph replayed after its warm-up run, a step launched ahead and dropped) gives the same
// state.  The convolution's history is a ring of `taps` positions, position p in place p mod taps, with the same
// property.
//
// Everything is float: decays, step sizes, softplus, exponentials, states and their sums.  Only the inputs that
// come out of a projection or a convolution may be 16-bit.
#include "common.cuh"

__device__ __forceinline__ float ik_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float ik_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ik_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ------------------------------------------------------------------ causal convolution
// y[p, c] = act(b[c] + sum_j w[j, c] * u[p - taps + 1 + j, c]), u = 0 before the sequence's start.  u of this step's
// tokens comes from x (row stride ldx), older ones from the ring.  w is tap-major [taps, C].
// inline_ring: every sequence brings one token, so the kernel also writes u[p] into the ring (nobody reads that place
// in this step); otherwise conv_ring_kernel does it afterwards.
template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                   float* __restrict__ ring, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ token_seq, const int* __restrict__ token_pos, TO* __restrict__ out,
                   int T, int C, int taps, int act, int inline_ring) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    ik_pdl_launch_dependents();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * C) return;
    const int t = (int)(idx / C), c = (int)(idx - (size_t)t * C);
    const int b = token_seq[t], pos = token_pos[t], first = cu_seqlens[b];
    const float* rg = ring ? ring + (size_t)slots[b] * taps * C : nullptr;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;                   // the input `back` positions ago
        if (back > pos) continue;                        // before the sequence's start
        float u;
        if (t - back >= first) u = x[(size_t)(t - back) * ldx + c];
        else u = rg[(size_t)((pos - back) % taps) * C + c];
        acc = fmaf(w[(size_t)j * C + c], u, acc);
    }
    if (inline_ring && ring) ring[((size_t)slots[b] * taps + pos % taps) * C + c] = x[(size_t)t * ldx + c];
    ik_st(out, idx, act ? ik_silu(acc) : acc);
}

// The same for four neighbouring channels per thread (channel counts and row distances that are multiples of four,
// aligned pointers): 16-byte accesses, and a token's few index computations once per four results.
template <typename TO>
__global__ void __launch_bounds__(256)
causal_conv4_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                    float* __restrict__ ring, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ token_seq, const int* __restrict__ token_pos, TO* __restrict__ out,
                    int T, int C, int taps, int act, int inline_ring) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    ik_pdl_launch_dependents();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4, t = blockIdx.x;
    if (c >= C) return;
    const int b = token_seq[t], pos = token_pos[t], first = cu_seqlens[b];
    const float* rg = ring ? ring + (size_t)slots[b] * taps * C : nullptr;
    float4 acc = bias ? ik_ld4(bias, c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        if (back > pos) continue;
        const float4 u = t - back >= first ? ik_ld4(x, (size_t)(t - back) * ldx + c) : ik_ld4(rg, (size_t)((pos - back) % taps) * C + c);
        const float4 wj = ik_ld4(w, (size_t)j * C + c);
        acc.x = fmaf(wj.x, u.x, acc.x); acc.y = fmaf(wj.y, u.y, acc.y); acc.z = fmaf(wj.z, u.z, acc.z); acc.w = fmaf(wj.w, u.w, acc.w);
    }
    if (inline_ring && ring) ik_st4(ring, ((size_t)slots[b] * taps + pos % taps) * C + c, ik_ld4(x, (size_t)t * ldx + c));
    if (act) { acc.x = ik_silu(acc.x); acc.y = ik_silu(acc.y); acc.z = ik_silu(acc.z); acc.w = ik_silu(acc.w); }
    ik_st4(out, (size_t)t * C + c, acc);
}

// The last `taps` inputs of every sequence go into its ring.
__global__ void __launch_bounds__(256)
conv_ring_kernel(const float* __restrict__ x, int ldx, float* __restrict__ ring, const int* __restrict__ slots,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens, int C, int taps) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.y;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b];
    const int n = min(taps, hi - lo);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n * C; i += gridDim.x * blockDim.x) {
        const int k = i / C, c = i - k * C;              // the k-th of the last n tokens
        const int t = hi - n + k, pos = end - n + k;
        ring[((size_t)slots[b] * taps + pos % taps) * C + c] = x[(size_t)t * ldx + c];
    }
}

IK_EXPORT int ik_causal_conv(const float* x, int ldx, const float* w, const float* bias, float* ring, const int* slots,
                             const int* cu_seqlens, const int* kv_lens, const int* token_seq, const int* token_pos,
                             void* out, int out_dtype, int T, int B, int C, int taps, int act, int one_token_each,
                             cudaStream_t stream) {
    if (T < 0 || B < 0 || C <= 0 || taps <= 0 || ldx < C || (taps > 1 && !ring)) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * C;
    const int blocks = (int)((total + 255) / 256);
    const int inl = one_token_each && taps > 1;
    const bool by4 = C % 4 == 0 && ldx % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (!bias || (uintptr_t)bias % 16 == 0) && (!ring || (uintptr_t)ring % 16 == 0);
    if (by4 && (out_dtype == IK_F32 || out_dtype == IK_BF16)) {
        const int threads = C / 4 >= 256 ? 256 : ((C / 4 + 31) / 32) * 32;
        const dim3 grid(T, (C / 4 + threads - 1) / threads);
        if (out_dtype == IK_F32)
            IK_RETURN_IF_ERROR(ik_launch(causal_conv4_kernel<float>, grid, threads, 0, stream, x, ldx, w, bias, ring, slots, cu_seqlens,
                                         token_seq, token_pos, (float*)out, T, C, taps, act, inl));
        else
            IK_RETURN_IF_ERROR(ik_launch(causal_conv4_kernel<__nv_bfloat16>, grid, threads, 0, stream, x, ldx, w, bias, ring, slots,
                                         cu_seqlens, token_seq, token_pos, (__nv_bfloat16*)out, T, C, taps, act, inl));
    } else if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(causal_conv_kernel<float>, blocks, 256, 0, stream, x, ldx, w, bias, ring, slots, cu_seqlens,
                                     token_seq, token_pos, (float*)out, T, C, taps, act, inl));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(causal_conv_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, ldx, w, bias, ring, slots,
                                     cu_seqlens, token_seq, token_pos, (__nv_bfloat16*)out, T, C, taps, act, inl));
    else
        return IK_BAD_ARGUMENT;
    if (taps > 1 && !inl) {
        const dim3 grid(min(64, (taps * C + 255) / 256), B);
        IK_RETURN_IF_ERROR(ik_launch(conv_ring_kernel, grid, 256, 0, stream, x, ldx, ring, slots, cu_seqlens, kv_lens, C, taps));
    }
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ selective scan
// Per channel c and state n:  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;  y_c = sum_n S[c, n] C_n + D_c u_c;
// out = y * silu(z).  dt = softplus(dt_raw + dt_bias).  B_n, C_n are columns of `bc` (row stride ldbc), z of `z`
// (row stride ldz).  L lanes (a power of two) share a channel: lane l holds states l, l + L, ... (NPT of them at most);
// their sums are added by shuffles in a fixed order.  One block row per sequence, tokens in order.
//
// The tokens go through shared memory in tiles: while a tile is computed, the next tile's inputs are on their way
// into registers; softplus and silu are applied when a tile is stored, by all threads at once, so that the
// token-by-token chain holds only the exponential and the multiply-adds.  What is computed for a token does not
// depend on where tiles begin.  FAST (16-bit inputs): exponentials and the gate's sigmoid are the hardware's
// approximations.
template <bool FAST> __device__ __forceinline__ float ik_silu_as(float x) {
    return FAST ? x * __frcp_rn(1.0f + __expf(-x)) : x / (1.0f + expf(-x));
}

// A load that is issued where it stands (the compiler may otherwise sink it to its first use, behind the tile's arithmetic).
__device__ __forceinline__ float ik_ld_now(const float* p) { float v; asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p)); return v; }
// The 16-bit value stays as it was loaded until ik_raw_float turns it into a float where it is used: a conversion next to
// the load would wait for the load.
__device__ __forceinline__ unsigned short ik_ld_now(const __nv_bfloat16* p) {
    unsigned short v;
    asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ik_raw_float(float v) { return v; }
__device__ __forceinline__ float ik_raw_float(unsigned short v) { return __uint_as_float((unsigned)v << 16); }
template <typename T> struct IkRaw { typedef float type; };
template <> struct IkRaw<__nv_bfloat16> { typedef unsigned short type; };
template <bool FAST> __device__ __forceinline__ float ik_softplus_as(float x) {
    return x > 20.0f ? x : (FAST ? __logf(1.0f + __expf(x)) : log1pf(expf(x)));
}

// NPT states a thread, L lanes a channel, TT tokens a tile: all fixed at compile time, so that the tile's layout and the
// sum over lanes are constants.  Lane l holds states l*NPT .. l*NPT + NPT - 1; the L*NPT >= N places beyond N are padding
// (A = 0, B = C = 0: they stay zero and add nothing), which spares every guard in the token loop.
// One state's step, S <- exp(dt a) S + dt x B.  16-bit path: float, with the hardware's exponential.  float32 path: the
// factor and the update are formed in double and rounded to float once, so that a step's error is half a unit in the last
// place and has no bias that could add up over thousands of steps (the state itself stays a float).
template <bool FAST> __device__ __forceinline__ float ik_scan_step(float S, float dt, float x, float a, float B) {
    if (FAST) return fmaf(__expf(dt * a), S, dt * x * B);
    return (float)fma(exp((double)dt * (double)a), (double)S, (double)dt * (double)x * (double)B);
}

template <typename TU, typename TO, bool FAST, int NPT, int L, int TT>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const TU* __restrict__ u, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                      const float* __restrict__ A, const float* __restrict__ bc, int ldbc, int b_off, int c_off,
                      const float* __restrict__ Dv, const float* __restrict__ z, int ldz, float* __restrict__ state,
                      const int* __restrict__ slots, const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                      TO* __restrict__ out, int inner, int N) {
    constexpr int CH = 128 / L, NPAD = L * NPT, W = 3 * CH + 2 * NPAD, PER_TILE = TT * W;
    constexpr int KX = (TT * CH + 127) / 128, KB = (TT * 2 * NPAD + 127) / 128;      // staged values a thread
    extern __shared__ __align__(16) float sm[];      // [2][TT][W]: x, dt, silu(z) per channel; B (padded), C (padded)
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(dt_raw);
    IK_AFTER_WAIT(bc);
    IK_AFTER_WAIT(z);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.y;
    const int l = threadIdx.x & (L - 1), ch = threadIdx.x / L;
    const int c0 = blockIdx.x * CH, c = c0 + ch;
    const bool live = c < inner;
    const int cc = live ? c : inner - 1;                     // idle lanes follow along (the shuffles need them)
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    if (hi <= lo) return;
    float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * inner * N + (size_t)cc * N;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * inner * N + (size_t)cc * N;
    float S[NPT], a[NPT];
    #pragma unroll
    for (int r = 0; r < NPT; r++) {
        const int n = l * NPT + r;
        a[r] = n < N ? A[(size_t)cc * N + n] : 0.f;
        S[r] = (n < N && start > 0) ? st_in[n] : 0.f;
    }
    const float dskip = Dv ? Dv[cc] : 0.f;
    typename IkRaw<TU>::type rx[KX];
    float rd[KX], rz[KX], rb[KB], bias_k[KX];
    #pragma unroll
    for (int k = 0; k < KX; k++) {
        const int col = c0 + ((threadIdx.x + k * 128) % CH);
        bias_k[k] = (dt_bias && col < inner) ? dt_bias[col] : 0.f;
    }
    auto fetch = [&](int t0) {
        #pragma unroll
        for (int k = 0; k < KX; k++) {
            const int e = threadIdx.x + k * 128, tt = e / CH, col = c0 + e % CH;
            const int t = min(t0 + tt, hi - 1);
            rx[k] = 0;
            rd[k] = rz[k] = 0.f;
            if (tt < TT && col < inner) {
                rx[k] = ik_ld_now(u + (size_t)t * inner + col);
                rd[k] = ik_ld_now(dt_raw + (size_t)t * inner + col);
                if (z) rz[k] = ik_ld_now(z + (size_t)t * ldz + col);
            }
        }
        #pragma unroll
        for (int k = 0; k < KB; k++) {
            const int e = threadIdx.x + k * 128, tt = e / (2 * NPAD), n2 = e % (2 * NPAD), n = n2 % NPAD;
            const int t = min(t0 + tt, hi - 1);
            rb[k] = 0.f;
            if (tt < TT && n < N) rb[k] = ik_ld_now(bc + (size_t)t * ldbc + (n2 < NPAD ? b_off : c_off) + n);
        }
    };
    auto store = [&](int buf) {
        float* tile = sm + buf * PER_TILE;
        #pragma unroll
        for (int k = 0; k < KX; k++) {
            const int e = threadIdx.x + k * 128, tt = e / CH, w = e % CH;
            if (tt < TT) {
                tile[tt * W + w] = ik_raw_float(rx[k]);
                tile[tt * W + CH + w] = ik_softplus_as<FAST>(rd[k] + bias_k[k]);
                tile[tt * W + 2 * CH + w] = ik_silu_as<FAST>(rz[k]);
            }
        }
        #pragma unroll
        for (int k = 0; k < KB; k++) {
            const int e = threadIdx.x + k * 128, tt = e / (2 * NPAD), n2 = e % (2 * NPAD);
            if (tt < TT) tile[tt * W + 3 * CH + n2] = rb[k];
        }
    };
    fetch(lo);
    store(0);
    __syncthreads();
    int buf = 0;
    for (int t0 = lo; t0 < hi; t0 += TT, buf ^= 1) {
        if (t0 + TT < hi) fetch(t0 + TT);
        const int n_here = min(TT, hi - t0);
        const float* tile = sm + buf * PER_TILE;
        // the tile's tokens in order; a token's sum over this lane's states stays in a register, the lanes' sums are added
        // for the whole tile afterwards (the shuffles are off the token-by-token chain)
        float acc[TT];
        #pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            const float* row = tile + tt * W;
            const float dt = row[CH + ch], x = row[ch];
            float bv[NPT], cv[NPT];
            if (NPT % 4 == 0) {
                #pragma unroll
                for (int r = 0; r < NPT; r += 4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(row + 3 * CH + l * NPT + r);
                    const float4 c4 = *reinterpret_cast<const float4*>(row + 3 * CH + NPAD + l * NPT + r);
                    bv[r] = b4.x; bv[r + 1] = b4.y; bv[r + 2] = b4.z; bv[r + 3] = b4.w;
                    cv[r] = c4.x; cv[r + 1] = c4.y; cv[r + 2] = c4.z; cv[r + 3] = c4.w;
                }
            } else {
                #pragma unroll
                for (int r = 0; r < NPT; r++) { bv[r] = row[3 * CH + l * NPT + r]; cv[r] = row[3 * CH + NPAD + l * NPT + r]; }
            }
            float a0 = 0.f, a1 = 0.f;
            if (tt < n_here) {
                #pragma unroll
                for (int r = 0; r < NPT; r++) {
                    S[r] = ik_scan_step<FAST>(S[r], dt, x, a[r], bv[r]);
                    if (r & 1) a1 = fmaf(S[r], cv[r], a1);
                    else a0 = fmaf(S[r], cv[r], a0);
                }
            }
            acc[tt] = a0 + a1;
        }
        #pragma unroll
        for (int tt = 0; tt < TT; tt++) {
            float v = acc[tt];
            #pragma unroll
            for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (l == 0 && live && tt < n_here) {
                const float* row = tile + tt * W;
                float y = fmaf(dskip, row[ch], v);
                if (z) y *= row[2 * CH + ch];
                ik_st(out, (size_t)(t0 + tt) * inner + c, y);
            }
        }
        if (t0 + TT < hi) store(buf ^ 1);
        __syncthreads();
    }
    if (live) {
        #pragma unroll
        for (int r = 0; r < NPT; r++) {
            const int n = l * NPT + r;
            if (n < N) st_out[n] = S[r];
        }
    }
}

// One token per sequence (a decode step): no tiles; every thread reads its own inputs and its NPT states, advances them and
// writes them to the other parity's copy.  The arithmetic and its order are those of the kernel above, so a token gives
// the same float32 bits whichever kernel runs it.
template <typename TU, typename TO, bool FAST, int NPT, int L>
__global__ void __launch_bounds__(128)
selective_scan_decode_kernel(const TU* __restrict__ u, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                             const float* __restrict__ A, const float* __restrict__ bc, int ldbc, int b_off, int c_off,
                             const float* __restrict__ Dv, const float* __restrict__ z, int ldz, float* __restrict__ state,
                             const int* __restrict__ slots, const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                             TO* __restrict__ out, int inner, int N) {
    constexpr int CH = 128 / L;
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(dt_raw);
    IK_AFTER_WAIT(bc);
    IK_AFTER_WAIT(z);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.y, l = threadIdx.x & (L - 1), c = blockIdx.x * CH + threadIdx.x / L;
    const bool live = c < inner;
    const int cc = live ? c : inner - 1;
    const int t = cu_seqlens[b], end = kv_lens[b], start = end - 1;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * inner * N + (size_t)cc * N;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * inner * N + (size_t)cc * N;
    const float x = ik_ld(u, (size_t)t * inner + cc);
    const float dt = ik_softplus_as<FAST>(dt_raw[(size_t)t * inner + cc] + (dt_bias ? dt_bias[cc] : 0.f));
    const float* row = bc + (size_t)t * ldbc;
    float S[NPT], a0 = 0.f, a1 = 0.f;
    #pragma unroll
    for (int r = 0; r < NPT; r++) {
        const int n = l * NPT + r;
        if (n < N) {
            const float ar = A[(size_t)cc * N + n];
            S[r] = start > 0 ? st_in[n] : 0.f;
            S[r] = ik_scan_step<FAST>(S[r], dt, x, ar, row[b_off + n]);
            if (r & 1) a1 = fmaf(S[r], row[c_off + n], a1);
            else a0 = fmaf(S[r], row[c_off + n], a0);
            if (live) st_out[n] = S[r];
        }
    }
    float v = a0 + a1;
    #pragma unroll
    for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (l == 0 && live) {
        float y = fmaf(Dv ? Dv[cc] : 0.f, x, v);
        if (z) y *= ik_silu_as<FAST>(z[(size_t)t * ldz + cc]);
        ik_st(out, (size_t)t * inner + c, y);
    }
}

template <typename TU, typename TO, bool FAST>
static int launch_scan(const void* u, const float* dt_raw, const float* dt_bias, const float* A, const float* bc, int ldbc, int b_off,
                       int c_off, const float* Dv, const float* z, int ldz, float* state, const int* slots, const int* cu_seqlens,
                       const int* kv_lens, void* out, int B, int inner, int N, int one_token_each, cudaStream_t stream) {
    // four states a thread (eight from 65 states on), as many lanes a channel as that takes, tiles as long as a thread's
    // staging registers allow
#define IK_SCAN(NPT, L, TT)                                                                                                     \
    do {                                                                                                                        \
        constexpr int CH = 128 / (L), W = 3 * CH + 2 * (L) * (NPT);                                                             \
        const dim3 grid((inner + CH - 1) / CH, B);                                                                              \
        if (one_token_each)                                                                                                     \
            IK_RETURN_IF_ERROR(ik_launch(selective_scan_decode_kernel<TU, TO, FAST, NPT, L>, grid, 128, 0, stream, (const TU*)u, dt_raw,   \
                                         dt_bias, A, bc, ldbc, b_off, c_off, Dv, z, ldz, state, slots, cu_seqlens, kv_lens, (TO*)out,    \
                                         inner, N));                                                                            \
        else                                                                                                                    \
        IK_RETURN_IF_ERROR(ik_launch(selective_scan_kernel<TU, TO, FAST, NPT, L, TT>, grid, 128, (size_t)2 * (TT) * W * sizeof(float), stream, \
                                     (const TU*)u, dt_raw, dt_bias, A, bc, ldbc, b_off, c_off, Dv, z, ldz, state, slots, cu_seqlens,  \
                                     kv_lens, (TO*)out, inner, N));                                                             \
    } while (0)
    // up to 16 states, 16-bit path: two states a thread while four would leave the SMs with fewer than two warps a scheduler
    // (one 4,096-token prompt, 4,096 channels: 1.01 -> 0.88 ms).  The float32 path keeps one shape whatever the batch, so
    // that its sums never depend on what else a step brings.
    const bool two = FAST && (long long)((inner + 31) / 32) * B * 4 < 8LL * ik_sm_count();
    if (N <= 16 && two) IK_SCAN(2, 8, 16);
    else if (N <= 16) IK_SCAN(4, 4, 16);
    else if (N <= 32) IK_SCAN(4, 8, 16);
    else if (N <= 64) IK_SCAN(4, 16, 16);
    else if (N <= 128) IK_SCAN(8, 16, 8);
    else if (N <= 256) IK_SCAN(8, 32, 4);
    else return IK_UNSUPPORTED;
#undef IK_SCAN
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_selective_scan(const void* u, int u_dtype, const float* dt_raw, const float* dt_bias, const float* A,
                                const float* bc, int ldbc, int b_off, int c_off, const float* Dv, const float* z, int ldz,
                                float* state, const int* slots, const int* cu_seqlens, const int* kv_lens, void* out,
                                int out_dtype, int T, int B, int inner, int N, int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || inner <= 0 || N <= 0 || !state || b_off < 0 || c_off < 0 || ldbc < N) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    if (one_token_each && T != B) return IK_BAD_ARGUMENT;
#define IK_ARGS u, dt_raw, dt_bias, A, bc, ldbc, b_off, c_off, Dv, z, ldz, state, slots, cu_seqlens, kv_lens, out, B, inner, N, one_token_each, stream
    if (u_dtype == IK_F32 && out_dtype == IK_F32) return launch_scan<float, float, false>(IK_ARGS);
    if (u_dtype == IK_BF16 && out_dtype == IK_BF16) return launch_scan<__nv_bfloat16, __nv_bfloat16, true>(IK_ARGS);
    if (u_dtype == IK_F32 && out_dtype == IK_BF16) return launch_scan<float, __nv_bfloat16, false>(IK_ARGS);
    if (u_dtype == IK_BF16 && out_dtype == IK_F32) return launch_scan<__nv_bfloat16, float, true>(IK_ARGS);
#undef IK_ARGS
    return IK_BAD_ARGUMENT;
}

// ------------------------------------------------------------------ linear attention with a constant decay per head
// Per head h with decay a_h:  S <- a_h S + k v^T (S is dk x dv);  o = S^T q.  q, k, v are columns of the projections'
// output `p` (row stride ldp), each passed through silu when act is set (act 2: with the hardware's approximate
// exponential and reciprocal, for the 16-bit path).  A block holds 32 columns of one head's S for one sequence: thread
// (j, part) keeps rows part*R .. part*R + R - 1 of column j in registers, one warp per part, up to 16 of them.  The
// tokens go through shared memory in tiles (q, k and the block's 32 columns of v, activation applied when a tile is
// stored); while a tile is computed the next one is on its way into registers, every warp fetching whole token rows.
// The parts' sums of a column are added in part order, once per tile.  What is computed for a token does not depend on
// where tiles begin.  FULL: dk = parts * RMAX and RMAX is a multiple of 4: no row is guarded and q, k come from shared
// memory four at a time.
constexpr int LA_ROWS = 2;         // token rows a warp stages per tile, at most

// LA_PER_ROW: 32-wide pieces of a staged row (2 dk + 32 values): 9 up to dk = 128, 17 up to 256
template <int RMAX, bool FULL, int LA_PER_ROW>
__global__ void __launch_bounds__(512)
decay_attention_kernel(const float* __restrict__ p, int ldp, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                       float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ kv_lens, float* __restrict__ out, int H, int dk, int dv, int R, int act, int TT) {
    extern __shared__ __align__(16) float sm[];          // [2][TT][2 dk + 32]: q, k, v;  [2][TT][parts][32] partial sums
    ik_pdl_wait();
    IK_AFTER_WAIT(p);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, part = threadIdx.y, parts = blockDim.y;
    const int col0 = blockIdx.z * 32, col = col0 + j;
    const bool live = col < dv;
    const int ccol = live ? col : dv - 1;
    const int tid = part * 32 + j, nthreads = parts * 32, W = 2 * dk + 32, per_tile = TT * W;
    float* partial = sm + 2 * per_tile;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    if (hi <= lo) return;
    const float a = decay[h];
    const size_t per = (size_t)H * dk * dv;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * per + (size_t)h * dk * dv;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * per + (size_t)h * dk * dv;
    float S[RMAX];
    #pragma unroll
    for (int r = 0; r < RMAX; r++) {
        const int i = part * R + r;
        S[r] = (r < R && i < dk && start > 0) ? st_in[(size_t)i * dv + ccol] : 0.f;
    }
    // staging: warp `part` fetches token rows part, part + parts, ...; lane j the columns j, j + 32, ... of a row
    float regs[LA_ROWS][LA_PER_ROW];
    auto fetch = [&](int t0) {
        #pragma unroll
        for (int rr = 0; rr < LA_ROWS; rr++) {
            const int tt = part + parts * rr;
            const float* row = p + (size_t)min(t0 + tt, hi - 1) * ldp;
            #pragma unroll
            for (int kk = 0; kk < LA_PER_ROW; kk++) {
                const int w = j + 32 * kk;
                regs[rr][kk] = 0.f;
                if (tt >= TT || w >= W) continue;
                if (w < dk) regs[rr][kk] = row[q_off + h * dk + w];
                else if (w < 2 * dk) regs[rr][kk] = row[k_off + h * dk + w - dk];
                else if (col0 + w - 2 * dk < dv) regs[rr][kk] = row[v_off + h * dv + col0 + w - 2 * dk];
            }
        }
    };
    auto store = [&](int buf) {
        #pragma unroll
        for (int rr = 0; rr < LA_ROWS; rr++) {
            const int tt = part + parts * rr;
            #pragma unroll
            for (int kk = 0; kk < LA_PER_ROW; kk++) {
                const int w = j + 32 * kk;
                if (tt < TT && w < W) sm[buf * per_tile + tt * W + w] = regs[rr][kk];
            }
        }
        if (!act) return;
        // the activation on what this thread has just stored, in a loop that is not unrolled (one copy of its code)
        for (int tt = part; tt < TT; tt += parts) {
            float* row = sm + buf * per_tile + tt * W;
            #pragma unroll 1
            for (int w = j; w < W; w += 32) row[w] = act == 2 ? ik_silu_as<true>(row[w]) : ik_silu_as<false>(row[w]);
        }
    };
    fetch(lo);
    store(0);
    __syncthreads();
    int buf = 0;
    for (int t0 = lo; t0 < hi; t0 += TT, buf ^= 1) {
        if (t0 + TT < hi) fetch(t0 + TT);
        const int n_here = min(TT, hi - t0);
        for (int tt = 0; tt < n_here; tt++) {
            const float* q = sm + buf * per_tile + tt * W + part * R;
            const float* k = q + dk;
            const float v = sm[buf * per_tile + tt * W + 2 * dk + j];
            float acc0 = 0.f, acc1 = 0.f;
            if (FULL) {
                #pragma unroll
                for (int r = 0; r < RMAX; r += 4) {
                    const float4 kk = *reinterpret_cast<const float4*>(k + r), qq = *reinterpret_cast<const float4*>(q + r);
                    S[r] = fmaf(a, S[r], kk.x * v);         acc0 = fmaf(S[r], qq.x, acc0);
                    S[r + 1] = fmaf(a, S[r + 1], kk.y * v); acc1 = fmaf(S[r + 1], qq.y, acc1);
                    S[r + 2] = fmaf(a, S[r + 2], kk.z * v); acc0 = fmaf(S[r + 2], qq.z, acc0);
                    S[r + 3] = fmaf(a, S[r + 3], kk.w * v); acc1 = fmaf(S[r + 3], qq.w, acc1);
                }
            } else {
                #pragma unroll
                for (int r = 0; r < RMAX; r++) {
                    if (r < R && part * R + r < dk) {
                        S[r] = fmaf(a, S[r], k[r] * v);
                        if (r & 1) acc1 = fmaf(S[r], q[r], acc1);
                        else acc0 = fmaf(S[r], q[r], acc0);
                    }
                }
            }
            const float acc = acc0 + acc1;
            if (parts > 1) partial[((buf * TT + tt) * parts + part) * 32 + j] = acc;
            else if (live) out[(size_t)(t0 + tt) * H * dv + h * dv + col] = acc;
        }
        if (t0 + TT < hi) store(buf ^ 1);
        __syncthreads();
        if (parts > 1) {
            for (int e = tid; e < n_here * 32; e += nthreads) {
                const int tt = e >> 5, jj = e & 31;
                if (col0 + jj >= dv) continue;
                float o = 0.f;
                for (int pp = 0; pp < parts; pp++) o += partial[((buf * TT + tt) * parts + pp) * 32 + jj];
                out[(size_t)(t0 + tt) * H * dv + h * dv + col0 + jj] = o;
            }
        }
    }
    if (live) {
        #pragma unroll
        for (int r = 0; r < RMAX; r++) {
            const int i = part * R + r;
            if (r < R && i < dk) st_out[(size_t)i * dv + col] = S[r];
        }
    }
}

// One token per sequence (a decode step): no tiles and few registers, so that several blocks share an SM and the state
// streams.  q and k pass the activation once per block (shared memory), every thread advances its R rows of its column
// and writes them to the other parity's copy.  The arithmetic and its order are those of the kernel above.
template <int RMAX>
__global__ void __launch_bounds__(512)
decay_attention_decode_kernel(const float* __restrict__ p, int ldp, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                              float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                              const int* __restrict__ kv_lens, float* __restrict__ out, int H, int dk, int dv, int R, int act) {
    extern __shared__ __align__(16) float sm[];          // [2 dk] q, k;  [parts][32] partial sums
    ik_pdl_wait();
    IK_AFTER_WAIT(p);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, part = threadIdx.y, parts = blockDim.y;
    const int col0 = blockIdx.z * 32, col = col0 + j;
    const bool live = col < dv;
    const int ccol = live ? col : dv - 1;
    const int tid = part * 32 + j, nthreads = parts * 32;
    float* partial = sm + 2 * dk;
    const int t = cu_seqlens[b], end = kv_lens[b], start = end - 1;
    const size_t per = (size_t)H * dk * dv;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * per + (size_t)h * dk * dv;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * per + (size_t)h * dk * dv;
    float S[RMAX];
    #pragma unroll
    for (int r = 0; r < RMAX; r++) {
        const int i = part * R + r;
        S[r] = (r < R && i < dk && start > 0) ? st_in[(size_t)i * dv + ccol] : 0.f;
    }
    const float* row = p + (size_t)t * ldp;
    for (int e = tid; e < 2 * dk; e += nthreads) {
        const float x = e < dk ? row[q_off + h * dk + e] : row[k_off + h * dk + e - dk];
        sm[e] = act == 2 ? ik_silu_as<true>(x) : act ? ik_silu_as<false>(x) : x;
    }
    float v = row[v_off + h * dv + ccol];
    v = act == 2 ? ik_silu_as<true>(v) : act ? ik_silu_as<false>(v) : v;
    const float a = decay[h];
    __syncthreads();
    const float* q = sm + part * R;
    const float* k = q + dk;
    float acc0 = 0.f, acc1 = 0.f;
    #pragma unroll
    for (int r = 0; r < RMAX; r++) {
        if (r < R && part * R + r < dk) {
            S[r] = fmaf(a, S[r], k[r] * v);
            if (r & 1) acc1 = fmaf(S[r], q[r], acc1);
            else acc0 = fmaf(S[r], q[r], acc0);
            if (live) st_out[(size_t)(part * R + r) * dv + col] = S[r];
        }
    }
    const float acc = acc0 + acc1;
    if (parts == 1) {
        if (live) out[(size_t)t * H * dv + h * dv + col] = acc;
        return;
    }
    partial[part * 32 + j] = acc;
    __syncthreads();
    if (part == 0 && live) {
        float o = 0.f;
        for (int pp = 0; pp < parts; pp++) o += partial[pp * 32 + j];
        out[(size_t)t * H * dv + h * dv + col] = o;
    }
}

IK_EXPORT int ik_decay_attention(const float* p, int ldp, int q_off, int k_off, int v_off, const float* decay, float* state,
                                 const int* slots, const int* cu_seqlens, const int* kv_lens, float* out, int T, int B, int H,
                                 int dk, int dv, int act, int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || H <= 0 || dk <= 0 || dv <= 0 || !state || !decay) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    if (dk > 256) return IK_UNSUPPORTED;
    if (one_token_each && T != B) return IK_BAD_ARGUMENT;
    int parts = (dk + 7) / 8;                       // eight rows a thread ...
    if (parts > 16) parts = 16;                     // ... sixteen from 129 rows on
    const int R = (dk + parts - 1) / parts, W = 2 * dk + 32;
    int TT = LA_ROWS * parts;
    if (TT > 16) TT = 16;
    const bool full = dk == parts * R && (R == 8 || R == 16) && ldp % 4 == 0;
    const dim3 grid(B, H, (dv + 31) / 32), block(32, parts);
    if (one_token_each) {
        const size_t smem1 = (size_t)(2 * dk + parts * 32) * sizeof(float);
        if (R <= 8)
            IK_RETURN_IF_ERROR(ik_launch(decay_attention_decode_kernel<8>, grid, block, smem1, stream, p, ldp, q_off, k_off, v_off, decay, state,
                                         slots, cu_seqlens, kv_lens, out, H, dk, dv, R, act));
        else
            IK_RETURN_IF_ERROR(ik_launch(decay_attention_decode_kernel<16>, grid, block, smem1, stream, p, ldp, q_off, k_off, v_off, decay, state,
                                         slots, cu_seqlens, kv_lens, out, H, dk, dv, R, act));
        IK_LAUNCH_STATUS();
    }
    const size_t smem = (size_t)(2 * TT * W + 2 * TT * parts * 32) * sizeof(float);
    if (smem > 160 * 1024) return IK_UNSUPPORTED;
#define IK_LA(RMAX, FULL, PER_ROW)                                                                                               \
    do {                                                                                                                         \
        static bool raised = false;                                                                                              \
        if (smem > 48 * 1024 && !raised) {                                                                                       \
            IK_RETURN_IF_ERROR(cudaFuncSetAttribute(decay_attention_kernel<RMAX, FULL, PER_ROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                    160 * 1024));                                                                \
            raised = true;                                                                                                       \
        }                                                                                                                        \
        IK_RETURN_IF_ERROR(ik_launch(decay_attention_kernel<RMAX, FULL, PER_ROW>, grid, block, smem, stream, p, ldp, q_off, k_off, v_off, \
                                     decay, state, slots, cu_seqlens, kv_lens, out, H, dk, dv, R, act, TT));                      \
    } while (0)
    if (full && R == 8) IK_LA(8, true, 9);
    else if (full) IK_LA(16, true, 17);
    else if (R <= 8) IK_LA(8, false, 9);
    else IK_LA(16, false, 17);
#undef IK_LA
    IK_LAUNCH_STATUS();
}
