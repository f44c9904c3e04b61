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
    if (out_dtype == IK_F32)
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
// (row stride ldz).  L lanes share a channel: lane l holds states l, l + L, ...; their sums are added by shuffles in a
// fixed order.  One block row per sequence, tokens in order.
constexpr int SCAN_NPT = 8;        // states per thread

template <typename TU, typename TO>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const TU* __restrict__ u, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                      const float* __restrict__ A, const float* __restrict__ bc, int ldbc, int b_off, int c_off,
                      const float* __restrict__ Dv, const float* __restrict__ z, int ldz, float* __restrict__ state,
                      const int* __restrict__ slots, const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                      TO* __restrict__ out, int inner, int N, int L) {
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
    const int l = threadIdx.x & (L - 1);
    const int c = blockIdx.x * (128 / L) + threadIdx.x / L;
    const bool live = c < inner;
    const int cc = live ? c : inner - 1;                     // idle lanes follow along (the shuffles need them)
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * inner * N + (size_t)cc * N;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * inner * N + (size_t)cc * N;
    float S[SCAN_NPT], a[SCAN_NPT];
    #pragma unroll
    for (int r = 0; r < SCAN_NPT; r++) {
        const int n = l + L * r;
        a[r] = n < N ? A[(size_t)cc * N + n] : 0.f;
        S[r] = (n < N && start > 0) ? st_in[n] : 0.f;
    }
    const float bias = dt_bias ? dt_bias[cc] : 0.f, dskip = Dv ? Dv[cc] : 0.f;
    // the next token's inputs are asked for while this one is computed
    float xn = 0.f, dn = 0.f, zn = 0.f, Bn[SCAN_NPT], Cn[SCAN_NPT];
    auto fetch = [&](int t) {
        xn = ik_ld(u, (size_t)t * inner + cc);
        dn = dt_raw[(size_t)t * inner + cc];
        zn = z ? z[(size_t)t * ldz + cc] : 0.f;
        const float* row = bc + (size_t)t * ldbc;
        #pragma unroll
        for (int r = 0; r < SCAN_NPT; r++) {
            const int n = l + L * r;
            Bn[r] = n < N ? row[b_off + n] : 0.f;
            Cn[r] = n < N ? row[c_off + n] : 0.f;
        }
    };
    if (lo < hi) fetch(lo);
    for (int t = lo; t < hi; t++) {
        const float x = xn, zz = zn, dt = ik_softplus(dn + bias);
        float Bt[SCAN_NPT], Ct[SCAN_NPT];
        #pragma unroll
        for (int r = 0; r < SCAN_NPT; r++) { Bt[r] = Bn[r]; Ct[r] = Cn[r]; }
        if (t + 1 < hi) fetch(t + 1);
        const float dx = dt * x;
        float acc = 0.f;
        #pragma unroll
        for (int r = 0; r < SCAN_NPT; r++) {
            if (l + L * r < N) {
                S[r] = fmaf(expf(dt * a[r]), S[r], dx * Bt[r]);
                acc = fmaf(S[r], Ct[r], acc);
            }
        }
        for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l == 0 && live) {
            float y = fmaf(dskip, x, acc);
            if (z) y *= ik_silu(zz);
            ik_st(out, (size_t)t * inner + c, y);
        }
    }
    if (live && hi > lo) {
        #pragma unroll
        for (int r = 0; r < SCAN_NPT; r++) {
            const int n = l + L * r;
            if (n < N) st_out[n] = S[r];
        }
    }
}

IK_EXPORT int ik_selective_scan(const void* u, int u_dtype, const float* dt_raw, const float* dt_bias, const float* A,
                                const float* bc, int ldbc, int b_off, int c_off, const float* Dv, const float* z, int ldz,
                                float* state, const int* slots, const int* cu_seqlens, const int* kv_lens, void* out,
                                int out_dtype, int T, int B, int inner, int N, cudaStream_t stream) {
    if (T < 0 || B < 0 || inner <= 0 || N <= 0 || !state || b_off < 0 || c_off < 0 || ldbc < N) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    int L = 1;
    while (L * SCAN_NPT < N) L *= 2;
    if (L > 32) return IK_UNSUPPORTED;
    const dim3 grid((inner + 128 / L - 1) / (128 / L), B);
#define IK_SCAN(TU, TO)                                                                                                    \
    IK_RETURN_IF_ERROR(ik_launch(selective_scan_kernel<TU, TO>, grid, 128, 0, stream, (const TU*)u, dt_raw, dt_bias, A, bc, ldbc, \
                                 b_off, c_off, Dv, z, ldz, state, slots, cu_seqlens, kv_lens, (TO*)out, inner, N, L))
    if (u_dtype == IK_F32 && out_dtype == IK_F32) IK_SCAN(float, float);
    else if (u_dtype == IK_BF16 && out_dtype == IK_BF16) IK_SCAN(__nv_bfloat16, __nv_bfloat16);
    else if (u_dtype == IK_F32 && out_dtype == IK_BF16) IK_SCAN(float, __nv_bfloat16);
    else if (u_dtype == IK_BF16 && out_dtype == IK_F32) IK_SCAN(__nv_bfloat16, float);
    else return IK_BAD_ARGUMENT;
#undef IK_SCAN
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ linear attention with a constant decay per head
// Per head h with decay a_h:  S <- a_h S + k v^T (S is dk x dv);  o = S^T q.  q, k, v are columns of the projections'
// output `p` (row stride ldp), each passed through silu when act is set.  A block holds 32 columns of one head's S for
// one sequence: thread (j, part) keeps rows part*R .. part*R + R - 1 of column j in registers.  q and k of a token are
// staged in shared memory (two buffers: the next token's are fetched while this one is computed); the parts' sums
// of a column are added in part order.
constexpr int LA_RMAX = 32;

__global__ void __launch_bounds__(256)
decay_attention_kernel(const float* __restrict__ p, int ldp, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                       float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ kv_lens, float* __restrict__ out, int H, int dk, int dv, int R, int act) {
    extern __shared__ __align__(16) float sm[];          // [2][2 dk] q then k;  [2][parts][32] partial sums
    ik_pdl_wait();
    IK_AFTER_WAIT(p);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, part = threadIdx.y, parts = blockDim.y;
    const int col = blockIdx.z * 32 + j;
    const bool live = col < dv;
    const int ccol = live ? col : dv - 1;
    const int tid = part * 32 + j, nthreads = parts * 32;
    float* qk = sm;
    float* partial = sm + 4 * dk;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    if (hi <= lo) return;
    const float a = decay[h];
    const size_t per = (size_t)H * dk * dv;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * per + (size_t)h * dk * dv;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * per + (size_t)h * dk * dv;
    float S[LA_RMAX];
    #pragma unroll
    for (int r = 0; r < LA_RMAX; r++) {
        const int i = part * R + r;
        S[r] = (r < R && i < dk && start > 0) ? st_in[(size_t)i * dv + ccol] : 0.f;
    }
    // staging: element e < dk is q_e, dk <= e < 2 dk is k_(e - dk)
    auto stage = [&](int t, int buf) {
        const float* row = p + (size_t)t * ldp;
        for (int e = tid; e < 2 * dk; e += nthreads) {
            float v = e < dk ? row[q_off + h * dk + e] : row[k_off + h * dk + e - dk];
            qk[buf * 2 * dk + e] = act ? ik_silu(v) : v;
        }
    };
    stage(lo, 0);
    float vn = p[(size_t)lo * ldp + v_off + h * dv + ccol];
    __syncthreads();
    for (int t = lo; t < hi; t++) {
        const int buf = (t - lo) & 1;
        const float v = act ? ik_silu(vn) : vn;
        if (t + 1 < hi) {
            vn = p[(size_t)(t + 1) * ldp + v_off + h * dv + ccol];
            stage(t + 1, buf ^ 1);
        }
        const float* q = qk + buf * 2 * dk + part * R;
        const float* k = q + dk;
        float acc = 0.f;
        #pragma unroll
        for (int r = 0; r < LA_RMAX; r++) {
            if (r < R && part * R + r < dk) {
                S[r] = fmaf(a, S[r], k[r] * v);
                acc = fmaf(S[r], q[r], acc);
            }
        }
        if (parts > 1) partial[(buf * parts + part) * 32 + j] = acc;
        __syncthreads();
        if (part == 0 && live) {
            float o = acc;
            for (int pp = 1; pp < parts; pp++) o += partial[(buf * parts + pp) * 32 + j];
            out[(size_t)t * H * dv + h * dv + col] = o;
        }
    }
    if (live) {
        #pragma unroll
        for (int r = 0; r < LA_RMAX; r++) {
            const int i = part * R + r;
            if (r < R && i < dk) st_out[(size_t)i * dv + col] = S[r];
        }
    }
}

IK_EXPORT int ik_decay_attention(const float* p, int ldp, int q_off, int k_off, int v_off, const float* decay, float* state,
                                 const int* slots, const int* cu_seqlens, const int* kv_lens, float* out, int T, int B, int H,
                                 int dk, int dv, int act, cudaStream_t stream) {
    if (T < 0 || B < 0 || H <= 0 || dk <= 0 || dv <= 0 || !state || !decay) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    const int parts = (dk + LA_RMAX - 1) / LA_RMAX;
    if (parts > 8) return IK_UNSUPPORTED;
    const int R = (dk + parts - 1) / parts;
    const dim3 grid(B, H, (dv + 31) / 32), block(32, parts);
    const size_t smem = (size_t)(4 * dk + 2 * parts * 32) * sizeof(float);
    IK_RETURN_IF_ERROR(ik_launch(decay_attention_kernel, grid, block, smem, stream, p, ldp, q_off, k_off, v_off, decay, state, slots,
                                 cu_seqlens, kv_lens, out, H, dk, dv, R, act));
    IK_LAUNCH_STATUS();
}
