// A selective state-space recurrence with a scalar decay per head (the Mamba-2 form), over the step's entries:
//
//     S_t = exp(-a_h dt_t) S_(t-1) + dt_t B_t x_t^T        S is [N state lanes][P value lanes] per (request, head)
//     y_t = S_t^T C_t + D_h x_t                            dt_t = softplus(dt_raw_t + dt_bias_h), never clamped
//
// Head h reads B and C of group h / (heads / groups).  The state is 32-bit, lives in a slot per request, starts at
// zero (the step's reset kernel) and is carried from step to step.  Everything that enters the recurrence here is
// 32-bit: dt from the projection's 32-bit sums, softplus, the decay and its exponential, the products into the state
// and out of it.  x, B and C come from the short convolution's output in the compute dtype.
//
// One token after the other is the only order the recurrence allows, so a long portion is cut into chunks of Q
// tokens that run side by side:
//   ssm_chunk_state   every chunk but an entry's last: the state it would end with had it started from zero, and
//                     the product of its decays;
//   ssm_chunk_carry   per (entry, head), chunk after chunk: start of chunk c + 1 = decay_c * start of chunk c + local_c,
//                     the first start being the request's state;
//   ssm_scan          every chunk from its true start: the outputs y, and the entry's last chunk leaves the
//                     request's new state.
// Entries of up to Q tokens (every decoded token) need the last kernel only.  A block is one (chunk, head, tile of
// value lanes); a thread holds up to 16 state lanes of one value lane in registers, L neighbouring lanes of a warp
// share a value lane and add their parts of y by shuffles.  B, C, x, dt of 16 tokens at a time are staged in shared
// memory.  The order of every sum depends on N and L only, not on how a prompt was cut.
//
//  * gated_group_norm   out = w * n_g(y * silu(z)): the recurrence's output gated by the z columns of the input
//                       projection, then cut into equal parts each divided by its own root mean square
#include "common.cuh"

namespace {

constexpr int NPT = 16;   // state lanes of one value lane that a thread holds at most
constexpr int PP = 4;     // value lanes a thread holds: what it reads of B and C from shared memory serves all of them
constexpr int NB = 16;    // tokens staged at a time

struct Rows {
    const float* p;       // [S][T][ld] 32-bit sums
    int S;
    long long s_stride;
    long long ld;
};

__device__ __forceinline__ float rows_at(const Rows& in, long long t, int c) {
    float v = 0.f;
    const float* p = in.p + t * in.ld + c;
    for (int s = 0; s < in.S; ++s) v += p[(long long)s * in.s_stride];
    return v;
}

__device__ __forceinline__ int entry_of_row(const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int t) {
    int lo = 0, hi = E;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (q_start[mid] <= t) lo = mid + 1;
        else hi = mid;
    }
    const int e = lo - 1;
    if (e < 0) return -1;
    return t - q_start[e] < q_len[e] ? e : -1;
}

struct SsmArgs {
    Rows u;               // the input projection's sums; column dt_col + h is head h's raw dt
    int dt_col;
    const void* xbc;      // [T][ldx] convolved and activated: x [heads P], then B [groups N], then C [groups N]
    long long ldx;
    const float* dt_bias; // [heads]
    const float* a;       // [heads] decay rates, exp(A_log)
    const float* D;       // [heads]
    float* state;         // [slots][heads][P][N]
    long long slot_stride;
    const int* q_start;
    const int* q_len;
    const int* slots;
    int E, heads, P, N, groups;
    int Q;                // tokens per chunk, a multiple of NB
    float* scratch;       // [chunks][heads][P][N]
    float* chunk_decay;   // [chunks][heads]
    float* y;             // [T][heads P]
    int L, npt, PT;       // threads per value lane (a power of two up to 32), 16-byte pieces of the state per thread, value lanes per block
};

// which entry and which of its chunks a chunk index is; false when there is no such chunk
__device__ __forceinline__ bool find_chunk(const SsmArgs& a, int blk, int& e, int& c, int& n, int& base) {
    int acc = 0;
    for (int i = 0; i < a.E; ++i) {
        const int k = (a.q_len[i] + a.Q - 1) / a.Q;
        if (blk < acc + k) {
            e = i; c = blk - acc; n = k; base = acc;
            return true;
        }
        acc += k;
    }
    return false;
}

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

__device__ __forceinline__ uint64_t pair_f32(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpair_f32(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pair(uint64_t x, uint64_t y, uint64_t z) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(x), "l"(y), "l"(z));
    return d;
}
__device__ __forceinline__ uint64_t mul_pair(uint64_t x, uint64_t y) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(x), "l"(y));
    return d;
}

// MODE 0: the local end state of a chunk from zero (no output); MODE 1: the outputs from the chunk's true start.
// L: threads that share a value lane (a power of two).  A thread's state lanes: up to four runs of four neighbours,
// n = 4 (l + L q) + k for q, k < 4, so that the L threads of a value lane read B and C as neighbouring 16-byte pieces
// (one conflict-free shared-memory load for all of them) and the state itself in 16-byte pieces too; the arithmetic
// runs on pairs of 32-bit lanes (fma.rn.f32x2: each lane an IEEE multiply-add).  Rows of B and C are padded with
// zeros to nq * L pieces, so a thread beyond the last state lane keeps zeros without being asked.
template <typename TX, int MODE, int L>
__global__ __launch_bounds__(256) void ssm_scan_kernel(SsmArgs a) {
    extern __shared__ float4 sm4[];
    pdl_trigger();
    pdl_wait();
    int e, c, n, base;
    if (!find_chunk(a, blockIdx.x, e, c, n, base)) return;
    if (MODE == 0 && (n <= 1 || c == n - 1)) return;
    const int h = blockIdx.y, g = h / (a.heads / a.groups);
    const int N = a.N, P = a.P, PT = a.PT;
    const int nq = a.npt;                    // 16-byte pieces a thread holds (1 to 4), the same for all
    const int N4 = nq * L;                   // 16-byte pieces of a padded row of B or C
    float4* Bs = sm4;                        // [NB][N4]
    float4* Cs = Bs + NB * N4;               // [NB][N4]
    float* xs = reinterpret_cast<float*>(Cs + NB * N4);   // [NB][PT] x
    float* dxs = xs + NB * PT;               // [NB][PT] dt * x
    float* ys = dxs + NB * PT;               // [NB][PT] outputs of the staged tokens
    float* dAs = ys + NB * PT;               // [NB]
    const int tid = threadIdx.x;
    const int pl = tid / L, l = tid % L;
    const int PG = PT / PP;                  // threads (of equal l) side by side: value lane k of thread pl is pl + k PG
    const int p0 = blockIdx.z * PT;
    const bool mine = pl < PG;
    const int inner = a.heads * P;
    const long long row0 = a.q_start[e] + (long long)c * a.Q;
    const int len = min(a.Q, a.q_len[e] - c * a.Q);
    const long long slot = a.slots[e];
    const bool vec = (N & 3) == 0;
    const size_t head_at = (size_t)h * P * N;

    uint64_t S2[PP][NPT / 2];
#pragma unroll
    for (int k = 0; k < PP; ++k)
#pragma unroll
        for (int i = 0; i < NPT / 2; ++i) S2[k][i] = 0ull;
    if (MODE == 1 && mine) {
        const float* src = (n > 1 ? a.scratch + (size_t)(base + c) * a.heads * P * N : a.state + slot * a.slot_stride) + head_at;
#pragma unroll
        for (int k = 0; k < PP; ++k) {
            const int p = p0 + pl + k * PG;
            if (p >= P) continue;
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                const int n0 = 4 * (l + L * q);
                if (q >= nq || n0 >= N) continue;
                const float* at = src + (size_t)p * N + n0;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (vec) v = *reinterpret_cast<const float4*>(at);
                else {
                    v.x = at[0];
                    if (n0 + 1 < N) v.y = at[1];
                    if (n0 + 2 < N) v.z = at[2];
                    if (n0 + 3 < N) v.w = at[3];
                }
                S2[k][2 * q] = pair_f32(v.x, v.y);
                S2[k][2 * q + 1] = pair_f32(v.z, v.w);
            }
        }
    }
    const float rate = a.a[h], bias = a.dt_bias[h], Dh = a.D[h];
    const TX* xbc = reinterpret_cast<const TX*>(a.xbc);
    float* Bf = reinterpret_cast<float*>(Bs);
    float* Cf = reinterpret_cast<float*>(Cs);
    const int Np = 4 * N4;
    // rows of B and C that can be fetched eight 16-bit values at a time
    const bool vec8 = sizeof(TX) == 2 && (N & 7) == 0 && (a.ldx & 7) == 0 && ((inner + g * N) & 7) == 0 && (((a.groups) * N) & 7) == 0 &&
                      ((uintptr_t)a.xbc & 15) == 0;
    float decay = 1.f;
    for (int j0 = 0; j0 < len; j0 += NB) {
        const int nb = min(NB, len - j0);
        __syncthreads();
        if (vec8) {
            const int per_row = Np >> 3;          // (N is a multiple of 8: no padding inside a piece of eight)
            for (int i = tid; i < nb * per_row; i += blockDim.x) {
                const int j = i / per_row, k = (i % per_row) * 8;
                float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0, c0 = b0, c1 = b0;
                if (k < N) {
                    const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(xbc) + (row0 + j0 + j) * a.ldx + inner + g * N + k;
                    const uint4 ub = *reinterpret_cast<const uint4*>(row);
                    const uint4 uc = *reinterpret_cast<const uint4*>(row + (size_t)a.groups * N);
                    b0 = make_float4(__uint_as_float(ub.x << 16), __uint_as_float(ub.x & 0xffff0000u), __uint_as_float(ub.y << 16), __uint_as_float(ub.y & 0xffff0000u));
                    b1 = make_float4(__uint_as_float(ub.z << 16), __uint_as_float(ub.z & 0xffff0000u), __uint_as_float(ub.w << 16), __uint_as_float(ub.w & 0xffff0000u));
                    c0 = make_float4(__uint_as_float(uc.x << 16), __uint_as_float(uc.x & 0xffff0000u), __uint_as_float(uc.y << 16), __uint_as_float(uc.y & 0xffff0000u));
                    c1 = make_float4(__uint_as_float(uc.z << 16), __uint_as_float(uc.z & 0xffff0000u), __uint_as_float(uc.w << 16), __uint_as_float(uc.w & 0xffff0000u));
                }
                Bs[j * N4 + (k >> 2)] = b0; Bs[j * N4 + (k >> 2) + 1] = b1;
                Cs[j * N4 + (k >> 2)] = c0; Cs[j * N4 + (k >> 2) + 1] = c1;
            }
        } else {
            for (int i = tid; i < nb * Np; i += blockDim.x) {
                const int j = i / Np, k = i % Np;
                const TX* row = xbc + (row0 + j0 + j) * a.ldx;
                Bf[i] = k < N ? to_f32(row[inner + g * N + k]) : 0.f;
                Cf[i] = k < N ? to_f32(row[inner + (a.groups + g) * N + k]) : 0.f;
            }
        }
        if (tid < nb) dAs[tid] = softplus_f(rows_at(a.u, row0 + j0 + tid, a.dt_col + h) + bias);   // dt for now
        __syncthreads();
        for (int i = tid; i < nb * PT; i += blockDim.x) {
            const int j = i / PT, k = i % PT;
            const float x = p0 + k < P ? to_f32(xbc[(row0 + j0 + j) * a.ldx + h * P + p0 + k]) : 0.f;
            xs[i] = x;
            dxs[i] = dAs[j] * x;
        }
        __syncthreads();
        if (tid < nb) dAs[tid] = expf(-rate * dAs[tid]);
        __syncthreads();
        for (int j = 0; j < nb; ++j) {
            const float dA = dAs[j];
            const uint64_t dA2 = pair_f32(dA, dA);
            uint64_t dtx2[PP], acc_lo[PP], acc_hi[PP];
#pragma unroll
            for (int k = 0; k < PP; ++k) {
                const float dtx = mine ? dxs[j * PT + pl + k * PG] : 0.f;
                dtx2[k] = pair_f32(dtx, dtx);
                acc_lo[k] = acc_hi[k] = 0ull;
            }
            const float4* Bj = Bs + j * N4 + l;
            const float4* Cj = Cs + j * N4 + l;
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                if (q < nq) {
                    const float4 bv = Bj[L * q];
                    const uint64_t b01 = pair_f32(bv.x, bv.y), b23 = pair_f32(bv.z, bv.w);
#pragma unroll
                    for (int k = 0; k < PP; ++k) {
                        S2[k][2 * q] = fma_pair(S2[k][2 * q], dA2, mul_pair(dtx2[k], b01));
                        S2[k][2 * q + 1] = fma_pair(S2[k][2 * q + 1], dA2, mul_pair(dtx2[k], b23));
                    }
                    if (MODE == 1) {
                        const float4 cv = Cj[L * q];
                        const uint64_t c01 = pair_f32(cv.x, cv.y), c23 = pair_f32(cv.z, cv.w);
#pragma unroll
                        for (int k = 0; k < PP; ++k) {
                            acc_lo[k] = fma_pair(S2[k][2 * q], c01, acc_lo[k]);
                            acc_hi[k] = fma_pair(S2[k][2 * q + 1], c23, acc_hi[k]);
                        }
                    }
                }
            }
            if (MODE == 1) {
#pragma unroll
                for (int k = 0; k < PP; ++k) {
                    float a0, a1, a2, a3;
                    unpair_f32(acc_lo[k], a0, a1);
                    unpair_f32(acc_hi[k], a2, a3);
                    float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
                    for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (l == 0 && mine) ys[j * PT + pl + k * PG] = fmaf(Dh, xs[j * PT + pl + k * PG], acc);
                }
            } else {
                decay *= dA;
            }
        }
        if (MODE == 1) {
            __syncthreads();
            for (int i = tid; i < nb * PT; i += blockDim.x) {
                const int j = i / PT, k = i % PT;
                if (p0 + k < P) a.y[(size_t)(row0 + j0 + j) * inner + h * P + p0 + k] = ys[i];
            }
        }
    }
    float* dst = nullptr;
    if (MODE == 0) {
        dst = a.scratch + (size_t)(base + c) * a.heads * P * N + head_at;
        if (tid == 0 && blockIdx.z == 0) a.chunk_decay[(size_t)(base + c) * a.heads + h] = decay;
    } else if (c == n - 1) {
        dst = a.state + slot * a.slot_stride + head_at;
    }
    if (dst != nullptr && mine) {
#pragma unroll
        for (int k = 0; k < PP; ++k) {
            const int p = p0 + pl + k * PG;
            if (p >= P) continue;
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
                const int n0 = 4 * (l + L * q);
                if (q >= nq || n0 >= N) continue;
                float* at = dst + (size_t)p * N + n0;
                float4 v;
                unpair_f32(S2[k][2 * q], v.x, v.y);
                unpair_f32(S2[k][2 * q + 1], v.z, v.w);
                if (vec) *reinterpret_cast<float4*>(at) = v;
                else {
                    at[0] = v.x;
                    if (n0 + 1 < N) at[1] = v.y;
                    if (n0 + 2 < N) at[2] = v.z;
                    if (n0 + 3 < N) at[3] = v.w;
                }
            }
        }
    }
}

// grid (entries, heads, slices of the head's P x N state elements): a thread an element, chunk after chunk; the next
// chunk's local state is asked for before this chunk's start is stored
__global__ void ssm_chunk_carry_kernel(SsmArgs a) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.x, h = blockIdx.y;
    const int n = (a.q_len[e] + a.Q - 1) / a.Q;
    if (n <= 1) return;
    int base = 0;
    for (int i = 0; i < e; ++i) base += (a.q_len[i] + a.Q - 1) / a.Q;
    const size_t per_head = (size_t)a.P * a.N, per_chunk = per_head * a.heads;
    const size_t i = (size_t)blockIdx.z * blockDim.x + threadIdx.x;
    if (i >= per_head) return;
    float S = a.state[(long long)a.slots[e] * a.slot_stride + h * per_head + i];
    float* at = a.scratch + (size_t)base * per_chunk + h * per_head + i;
    const float* dec = a.chunk_decay + (size_t)base * a.heads + h;
    float local = *at;
    for (int c = 0; c < n; ++c) {
        const float next = c + 1 < n - 1 ? at[per_chunk] : 0.f;
        *at = S;
        if (c < n - 1) S = fmaf(dec[(size_t)c * a.heads], S, local);
        local = next;
        at += per_chunk;
    }
}

// grid (rows, parts): out[t, c] = w[c] * v / sqrt(mean over the part of v^2 + eps), v = y[t, c] * silu(z[t, c])
template <typename TOUT>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, Rows z, const float* __restrict__ w, float eps,
                                        const int* __restrict__ q_start, const int* __restrict__ q_len, int E, int C, int gs,
                                        TOUT* __restrict__ out) {
    extern __shared__ float vals[];   // [gs] then 33 floats
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, c0 = blockIdx.y * gs;
    if (entry_of_row(q_start, q_len, E, t) < 0) return;
    float ss = 0.f;
    for (int k = threadIdx.x; k < gs; k += blockDim.x) {
        const float zz = rows_at(z, t, c0 + k);
        const float v = y[(size_t)t * C + c0 + k] * (zz / (1.f + expf(-zz)));
        vals[k] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, vals + gs);
    const float mul = 1.f / sqrtf(ss / (float)gs + eps);
    for (int k = threadIdx.x; k < gs; k += blockDim.x)
        out[(size_t)t * C + c0 + k] = from_f32<TOUT>(vals[k] * mul * w[c0 + k]);
}

// the same with four channels a thread, the part's values held in registers
template <typename TOUT, int VPT>
__global__ __launch_bounds__(1024) void gated_group_norm_vec_kernel(const float* __restrict__ y, Rows z, const float* __restrict__ w,
                                                                    float eps, const int* __restrict__ q_start,
                                                                    const int* __restrict__ q_len, int E, int C, int gs,
                                                                    TOUT* __restrict__ out) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, c0 = blockIdx.y * gs;
    if (entry_of_row(q_start, q_len, E, t) < 0) return;
    const int nv = gs >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        if (idx < nv) {
            const int c = c0 + 4 * idx;
            float4 zz = make_float4(0.f, 0.f, 0.f, 0.f);
            const float* zp = z.p + (long long)t * z.ld + c;
            for (int s = 0; s < z.S; ++s) {
                const float4 a = *reinterpret_cast<const float4*>(zp + (long long)s * z.s_stride);
                zz.x += a.x; zz.y += a.y; zz.z += a.z; zz.w += a.w;
            }
            const float4 yy = *reinterpret_cast<const float4*>(y + (size_t)t * C + c);
            v[k] = make_float4(yy.x * (zz.x / (1.f + expf(-zz.x))), yy.y * (zz.y / (1.f + expf(-zz.y))),
                               yy.z * (zz.z / (1.f + expf(-zz.z))), yy.w * (zz.w / (1.f + expf(-zz.w))));
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float mul = 1.f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        if (idx < nv) {
            const int c = c0 + 4 * idx;
            const float4 g = *reinterpret_cast<const float4*>(w + c);
            const float4 o = make_float4(v[k].x * mul * g.x, v[k].y * mul * g.y, v[k].z * mul * g.z, v[k].w * mul * g.w);
            if (sizeof(TOUT) == 4) *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)t * C + c) = o;
            else {
                const __nv_bfloat162 a = __floats2bfloat162_rn(o.x, o.y), b = __floats2bfloat162_rn(o.z, o.w);
                uint2 u;
                u.x = *reinterpret_cast<const uint32_t*>(&a);
                u.y = *reinterpret_cast<const uint32_t*>(&b);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)t * C + c) = u;
            }
        }
    }
}

// a launch of one build of the scan kernel; shared memory beyond the default 48 KB has to be asked for per build (all
// builds have one function type, so nothing is remembered here: the call is a few microseconds of host time)
template <typename K>
int scan_launch(K kern, dim3 grid, int threads, size_t smem, cudaStream_t stream, const SsmArgs& args) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        vcb_set_error("ssm_scan: %zu bytes of shared memory refused", smem);
        return -2;
    }
    launch_pdl(kern, grid, dim3(threads), smem, stream, args);
    return 0;
}

}  // namespace

// The three kernels of the recurrence.  u: the input projection's sums [S][T][ld] (dt of head h in column dt_col + h);
// xbc [T][ldx] of xbc_dtype; state [slots][heads][P][N]; y [T][heads P] 32-bit.  n_chunks: how many chunks of Q tokens the
// step's entries can have (the sum over entries of ceil(q_len / Q), or more); multi: whether any entry may have more
// than one chunk (then scratch [n_chunks][heads][P][N] and chunk_decay [n_chunks][heads] are needed).
VCB_API int vcb_ssm_scan(const float* u, int S, long long s_stride, long long ld, int dt_col, const void* xbc, int xbc_dtype,
                         long long ldx, const float* dt_bias, const float* a_rate, const float* D, float* state,
                         long long slot_stride, const int* q_start, const int* q_len, const int* slots, int E, int heads, int P,
                         int N, int groups, int Q, int n_chunks, int multi, float* scratch, float* chunk_decay, float* y,
                         cudaStream_t stream) {
    if (n_chunks == 0 || E == 0) return 0;
    VCB_CHECK_ARG(heads > 0 && groups > 0 && heads % groups == 0, "ssm_scan: %d heads are not a multiple of %d groups", heads, groups);
    VCB_CHECK_ARG(N >= 1 && N <= NPT * 32, "ssm_scan: %d state lanes (1 to %d)", N, NPT * 32);
    VCB_CHECK_ARG(P >= 1 && Q >= NB && Q % NB == 0, "ssm_scan: bad sizes P=%d Q=%d", P, Q);
    VCB_CHECK_ARG(!multi || (scratch != nullptr && chunk_decay != nullptr), "ssm_scan: chunks need their scratch");
    VCB_CHECK_ARG(n_chunks <= 0x7fffffff / 1 && heads <= 65535 && E <= 65535, "ssm_scan: too many heads or entries");
    const int N4 = (N + 3) / 4;
    int L = 1;
    while (L * (NPT / 4) < N4) L <<= 1;
    const int nq = (N4 + L - 1) / L;          // 16-byte pieces of the state a thread holds
    int PG = 256 / L;                          // threads side by side, each with PP value lanes
    if (PG > 32) PG = 32;
    if (PG * PP > P) PG = (P + PP - 1) / PP;
    const int PT = PG * PP;                    // value lanes per block
    const int threads = (PG * L + 31) / 32 * 32;
    const int ptiles = (P + PT - 1) / PT;
    VCB_CHECK_ARG(ptiles <= 65535, "ssm_scan: too many tiles of value lanes");
    SsmArgs args{Rows{u, S < 1 ? 1 : S, s_stride, ld}, dt_col, xbc, ldx, dt_bias, a_rate, D, state, slot_stride, q_start, q_len,
                 slots, E, heads, P, N, groups, Q, scratch, chunk_decay, y, L, nq, PT};
    const size_t smem = ((size_t)2 * NB * 4 * nq * L + (size_t)3 * NB * PT + NB) * sizeof(float);
    VCB_CHECK_ARG(smem <= 200 * 1024, "ssm_scan: %d state lanes need more shared memory than a block has", N);
    const dim3 grid(n_chunks, heads, ptiles);
    const bool f32 = xbc_dtype == VCB_F32;
#define VCB_SSM(MODE, LL)                                                                                              \
    do {                                                                                                               \
        if (f32) { if (int rc = scan_launch(ssm_scan_kernel<float, MODE, LL>, grid, threads, smem, stream, args)) return rc; }            \
        else { if (int rc = scan_launch(ssm_scan_kernel<__nv_bfloat16, MODE, LL>, grid, threads, smem, stream, args)) return rc; }       \
    } while (0)
#define VCB_SSM_L(MODE)                                                                                                \
    switch (L) {                                                                                                       \
        case 1: VCB_SSM(MODE, 1); break;                                                                               \
        case 2: VCB_SSM(MODE, 2); break;                                                                               \
        case 4: VCB_SSM(MODE, 4); break;                                                                               \
        case 8: VCB_SSM(MODE, 8); break;                                                                               \
        case 16: VCB_SSM(MODE, 16); break;                                                                             \
        default: VCB_SSM(MODE, 32); break;                                                                             \
    }
    if (multi) {
        VCB_SSM_L(0)
        VCB_CHECK_LAUNCH("ssm_chunk_state");
        launch_pdl(ssm_chunk_carry_kernel, dim3(E, heads, (unsigned)(((size_t)P * N + 255) / 256)), dim3(256), 0, stream, args);
        VCB_CHECK_LAUNCH("ssm_chunk_carry");
    }
    VCB_SSM_L(1)
#undef VCB_SSM_L
#undef VCB_SSM
    VCB_CHECK_LAUNCH("ssm_scan");
    return 0;
}

// y [T][C] 32-bit; z: 32-bit sums [S][T][ld] whose first C columns gate y; w [C]; parts equal pieces of the row
VCB_API int vcb_gated_group_norm(const float* y, const float* z, int S, long long s_stride, long long ld, const float* w,
                                 float eps, const int* q_start, const int* q_len, int E, int T, int C, int parts, void* out,
                                 int out_dtype, cudaStream_t stream) {
    if (T == 0 || C == 0) return 0;
    VCB_CHECK_ARG(parts >= 1 && C % parts == 0 && parts <= 65535, "gated_group_norm: %d channels in %d parts", C, parts);
    const int gs = C / parts;
    Rows rz{z, S < 1 ? 1 : S, s_stride, ld};
    if (gs % 4 == 0 && gs / 4 <= 4096 && (uintptr_t)y % 16 == 0 && (uintptr_t)z % 16 == 0 && ld % 4 == 0 && (S <= 1 || s_stride % 4 == 0) &&
        (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 && C % 4 == 0) {
        const int nv = gs / 4;
        const int vpt = nv <= 256 ? 1 : (nv <= 2048 ? 2 : 4);
        const int threads4 = ((nv + vpt - 1) / vpt + 31) / 32 * 32;
#define VCB_GGN(TOUT, V) launch_pdl(gated_group_norm_vec_kernel<TOUT, V>, dim3(T, parts), dim3(threads4), 0, stream, y, rz, w, eps, q_start, q_len, E, C, gs, (TOUT*)out)
        if (out_dtype == VCB_F32) { if (vpt == 1) VCB_GGN(float, 1); else if (vpt == 2) VCB_GGN(float, 2); else VCB_GGN(float, 4); }
        else { if (vpt == 1) VCB_GGN(__nv_bfloat16, 1); else if (vpt == 2) VCB_GGN(__nv_bfloat16, 2); else VCB_GGN(__nv_bfloat16, 4); }
#undef VCB_GGN
        VCB_CHECK_LAUNCH("gated_group_norm");
        return 0;
    }
    const size_t smem = ((size_t)gs + 64) * sizeof(float);
    VCB_CHECK_ARG(smem <= 200 * 1024, "gated_group_norm: parts of %d channels are too long", gs);
    const int threads = gs >= 2048 ? 1024 : (gs >= 512 ? 512 : 256);
    if (out_dtype == VCB_F32) {
        auto kern = gated_group_norm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(kern, dim3(T, parts), dim3(threads), smem, stream, y, rz, w, eps, q_start, q_len, E, C, gs, (float*)out);
    } else {
        auto kern = gated_group_norm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_pdl(kern, dim3(T, parts), dim3(threads), smem, stream, y, rz, w, eps, q_start, q_len, E, C, gs, (__nv_bfloat16*)out);
    }
    VCB_CHECK_LAUNCH("gated_group_norm");
    return 0;
}
