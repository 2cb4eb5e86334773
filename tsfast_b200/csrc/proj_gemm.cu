// Boundary projections of the diagonal-scan layers (LRU / S5) on the 5th-generation tensor cores:
//   C[M, N] = A1[M, K1] * B1[N, K1]^T  (+ A2[M, K2] * B2[N, K2]^T),   float32 in, float32 out.
// M is the token axis (batch x time, hundreds of thousands of rows), K and N are feature widths
// (tens to hundreds), so each product is a skinny GEMM whose cost is reading A and writing C once;
// the only reason it is slow as a float32 SIMT GEMM is arithmetic.  Here the arithmetic runs as
// tcgen05.mma.kind::tf32 with float32-faithful numerics: every operand is split x = hi + lo with hi
// the value rounded to TF32 (10 mantissa bits) and lo the rounded remainder, and the product is
// accumulated in float32 in tensor memory as  lo*hi + hi*lo + hi*hi  (the dropped lo*lo term is below
// 2^-22 relative).
//
// One CTA (128 threads) computes one 128 x 128 tile of C:
//   * thread 0 asks the TMA unit for the next K-block (32 floats = one 128-byte swizzle row) of A and
//     of the two halves of B, which land in shared memory in the 128-byte-swizzled K-major layout the
//     tensor core reads (cp.async.bulk.tensor, completion on an mbarrier);
//   * all threads split the A block in place into hi and lo (elementwise, so the swizzle is irrelevant);
//   * thread 0 issues the 4 x 3 MMAs of the block (K = 8 per instruction) and commits them to a second
//     mbarrier; the accumulator [128 lanes x 128 columns] lives in tensor memory;
//   * after the last block each warp reads its 32 lanes with tcgen05.ld, stages them in shared memory
//     and stores whole 512-byte rows.
// Shared memory per CTA is 64 KB and the accumulator 128 of the 512 tensor-memory columns, so three
// CTAs share an SM and overlap one another's copy, split, MMA and store phases.
// The weights' halves are prepared once per call by split_weights_kernel into the caller's workspace.
// Every wait on an mbarrier is bounded; a wait that runs out records B200_ERR_TIMEOUT in the
// workspace header, and the CTA still frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace b200 {

constexpr int kBM = 128;       // rows of C per CTA (= tensor-memory lanes)
constexpr int kBN = 128;       // columns of C per CTA (= tensor-memory columns, MMA N)
constexpr int kBK = 32;        // floats per K-block: one 128-byte swizzle row
constexpr int kTileBytes = kBM * kBK * 4;  // 16 KB: one operand block
constexpr int kGemmSmem = 4 * kTileBytes + 1024;  // A(hi), A lo, B hi, B lo + alignment slack
constexpr int kWaitLimit = 200000;  // polls of an mbarrier (about 100 ns apart) before a wait gives up: tens of ms

struct ProjArgs {
    float* C;
    const float* bias;  // [N] added to every row, or null
    long long ldc;
    long long M, N;
    int kb1, kb2;  // K-blocks of the first and of the second product
    int tma_c;     // C rows are 16-byte aligned: the pipelined kernel stores it with TMA
    WsHeader* hdr;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false when the poll limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// TMA store of a [rows x 32 floats] box from (128-byte-swizzled) shared memory; rows and columns past
// the end of the tensor are clipped.  Bulk stores are tracked per issuing thread in groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
                 "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {  // at most N of this thread's store groups still reading shared memory
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand block in the 128-byte-swizzled layout: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major), 16 B
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;             // descriptor version
    d |= (uint64_t)2 << 61;             // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B TF32, both K-major, M = 128, N = kBN.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
// A operand read from tensor memory (lane = row, one column per TF32 element), B from shared memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive columns of this thread's lane <- 16 registers
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// x = hi + lo (+ a remainder below 2^-22 |x|): hi is x rounded to the nearest TF32 value (10 mantissa bits)
// and lo the rounded difference, so both halves are exactly what the tensor core will read and the
// rounding errors carry no common sign
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = round_tf32(x);
    lo = round_tf32(x - hi);
}

// B[N, K] (row pitch ldb) -> hi[N, Kp], lo[N, Kp] with Kp = K rounded up to 4 (16-byte row pitch for TMA)
__global__ void split_weights_kernel(const float* __restrict__ B, long long ldb, long long N, long long K, long long Kp,
                                     float* __restrict__ hi, float* __restrict__ lo) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * Kp) return;
    const long long r = i / Kp, c = i - r * Kp;
    float h = 0.f, l = 0.f;
    if (c < K) split_tf32(B[r * ldb + c], h, l);
    hi[i] = h;
    lo[i] = l;
}

__global__ void __launch_bounds__(128, 3)
proj_gemm_kernel(const __grid_constant__ CUtensorMap mapA1, const __grid_constant__ CUtensorMap mapB1hi,
                 const __grid_constant__ CUtensorMap mapB1lo, const __grid_constant__ CUtensorMap mapA2,
                 const __grid_constant__ CUtensorMap mapB2hi, const __grid_constant__ CUtensorMap mapB2lo,
                 const ProjArgs p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_tma, bar_mma;
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    // 1024-byte aligned operand blocks (the swizzle pattern repeats every 1024 bytes)
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* sA = reinterpret_cast<float*>(base);
    float* sAlo = reinterpret_cast<float*>(base + kTileBytes);
    float* sBhi = reinterpret_cast<float*>(base + 2 * kTileBytes);
    float* sBlo = reinterpret_cast<float*>(base + 3 * kTileBytes);

    const long long n_tiles = (p.N + kBN - 1) / kBN;
    const long long m_tile = blockIdx.x / n_tiles, n_tile = blockIdx.x - m_tile * n_tiles;
    const int row0 = (int)(m_tile * kBM), col0 = (int)(n_tile * kBN);

    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 1) {  // one warp allocates the accumulator columns and gives up the right to allocate more
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kBN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    // `ok` is uniform over the CTA (it comes out of a barrier vote), so a wait that ran out takes every
    // thread out of the loop together and no barrier is left half-attended
    int ok = 1;
    const int nkb = p.kb1 + p.kb2;
    for (int kb = 0; kb < nkb && ok; ++kb) {
        const uint32_t parity = (uint32_t)(kb & 1);
        if (tid == 0) {
            const bool first = kb < p.kb1;
            const int kx = (first ? kb : kb - p.kb1) * kBK;
            mbar_expect_tx(&bar_tma, 3 * kTileBytes);
            tma_load_2d(sA, first ? &mapA1 : &mapA2, kx, row0, &bar_tma);
            tma_load_2d(sBhi, first ? &mapB1hi : &mapB2hi, kx, col0, &bar_tma);
            tma_load_2d(sBlo, first ? &mapB1lo : &mapB2lo, kx, col0, &bar_tma);
        }
        const int landed = mbar_wait(&bar_tma, parity) ? 1 : 0;
        // split the A block: hi in place, lo beside it (same swizzled position)
#pragma unroll
        for (int j = 0; j < kTileBytes / 16 / 128; ++j) {
            float4 x = reinterpret_cast<float4*>(sA)[j * 128 + tid];
            float4 h, l;
            split_tf32(x.x, h.x, l.x), split_tf32(x.y, h.y, l.y), split_tf32(x.z, h.z, l.z), split_tf32(x.w, h.w, l.w);
            reinterpret_cast<float4*>(sA)[j * 128 + tid] = h;
            reinterpret_cast<float4*>(sAlo)[j * 128 + tid] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        ok = __syncthreads_and(landed);
        if (ok) {
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dA = umma_desc_k_sw128(smem_u32(sA)), dAl = umma_desc_k_sw128(smem_u32(sAlo));
                const uint64_t dBh = umma_desc_k_sw128(smem_u32(sBhi)), dBl = umma_desc_k_sw128(smem_u32(sBlo));
#pragma unroll
                for (int k = 0; k < kBK / 8; ++k) {  // 8 floats = 32 bytes per MMA along K: +2 in 16-byte units
                    const uint64_t adv = (uint64_t)(2 * k);
                    umma_tf32(tmem_d, dAl + adv, dBh + adv, (kb | k) != 0);
                    umma_tf32(tmem_d, dA + adv, dBl + adv, 1u);
                    umma_tf32(tmem_d, dA + adv, dBh + adv, 1u);
                }
                umma_commit(&bar_mma);
            }
            // the MMAs have read the blocks once this completes: only then may they be overwritten
            ok = __syncthreads_and(mbar_wait(&bar_mma, parity) ? 1 : 0);
        }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (ok) {
        // epilogue: warp w owns accumulator lanes (rows) 32w .. 32w+31; 32 columns at a time go through a
        // padded shared-memory patch so that every store instruction writes whole 128-byte row pieces
        float* patch = reinterpret_cast<float*>(base) + wid * (32 * 36);
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
            float v[32];
            tmem_ld32(tmem_d + ((uint32_t)(wid * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(patch + lane * 36 + q * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            __syncwarp();
            const int cc = (lane & 7) * 4;  // 8 lanes cover one row piece of 32 columns
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                const int r = rr * 4 + (lane >> 3);
                const long long grow = (long long)row0 + wid * 32 + r;
                const long long gcol = (long long)col0 + c * 32 + cc;
                if (grow < p.M && gcol < p.N) {
                    float4 o = *reinterpret_cast<const float4*>(patch + r * 36 + cc);
                    if (p.bias != nullptr) {
                        o.x += p.bias[gcol];
                        if (gcol + 1 < p.N) o.y += p.bias[gcol + 1];
                        if (gcol + 2 < p.N) o.z += p.bias[gcol + 2];
                        if (gcol + 3 < p.N) o.w += p.bias[gcol + 3];
                    }
                    float* dst = p.C + grow * p.ldc + gcol;
                    if (gcol + 3 < p.N) {
                        __stcs(reinterpret_cast<float4*>(dst), o);
                    } else {
                        const float ov[4] = {o.x, o.y, o.z, o.w};
                        for (int e = 0; e < 4 && gcol + e < p.N; ++e) dst[e] = ov[e];
                    }
                }
            }
            __syncwarp();
        }
    } else if (tid == 0) {
        atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // give copies still in flight a bounded time to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kBN) : "memory");
    }
}


// ================================================================================ pipelined version
// The same product as proj_gemm_kernel with the phases of different K-blocks and tiles running at the
// same time.  A CTA is persistent (one per SM, tiles dealt round-robin) and its warps have fixed roles
// that talk through mbarriers over a ring of kStages operand stages and two accumulators:
//   warp 8   producer: waits for a free stage, asks the TMA unit for A, B-hi, B-lo of the next K-block;
//   warps 4-7 splitters: when a stage has landed, every thread reads ITS row of the A block from shared
//            memory (the swizzle makes that conflict-free), splits it in registers and writes hi and lo
//            into tensor memory (tcgen05.st), from where the MMAs take their A operand: the A block
//            crosses shared memory once instead of being rewritten there twice and re-read three times;
//   warp 9   issuer: when a stage is split, issues its 12 MMAs (A from tensor memory, B from shared
//            memory); their completion frees the stage, and after a tile's last K-block hands the
//            accumulator to the epilogue;
//   warps 0-3 epilogue: read the finished accumulator (tcgen05.ld, warp w owns lanes 32w..32w+31), give it
//            back as soon as it is in registers, add the bias, write 32 x 32 patches into shared memory
//            (128-byte swizzle, two patches alternating) and hand each to the TMA unit, which stores it
//            while the next one is being filled (rows not 16-byte aligned: plain row stores instead).
// So the copy of block k+2, the split of block k+1, the MMAs of block k and the store of the previous
// tile overlap.  Every wait is bounded; a wait that gives up raises a CTA-wide abort flag that all roles
// poll, so the CTA winds down together, frees its tensor memory and reports B200_ERR_TIMEOUT.
constexpr int kStages = 4;
constexpr int kStageBytes = 3 * kTileBytes;                       // A, B-hi, B-lo
constexpr int kTmemAcc = 2 * kBN;                                 // two accumulators ...
constexpr int kTmemCols = 512;                                    // ... then kStages x (32 hi + 32 lo) columns of A
constexpr int kPatchBytes = 4 * 2 * 32 * 32 * 4;                  // epilogue staging: two 32 x 32 patches per warp
constexpr int kWsSmem = kStages * kStageBytes + kPatchBytes + 1024;
constexpr int kWsThreads = 320;

struct WsBars {
    uint64_t full[kStages], ready[kStages], empty[kStages], acc_full[2], acc_empty[2], b_full;
};
#ifndef PROJ_RESIDENT
#define PROJ_RESIDENT 1
#endif
#ifndef PROJ_TMA_STORE
#define PROJ_TMA_STORE 1
#endif
constexpr int kResidentKb = 4;  // K-blocks of B (hi and lo) that fit beside the A ring: K <= 128

// RESIDENT (K <= 128, one product): a CTA keeps ONE column tile for all its row tiles, so the split
// weights of that tile (K/32 blocks of hi and lo, at most 128 KB) are fetched once and stay in shared
// memory, and a stage of the ring carries the 16 KB A block alone: a third of the shared-memory fill
// (measured: 4 % faster on 256 000 x 512 x 128; the rest of the shared-memory traffic, the three reads
// of B by the MMAs and the epilogue's staging, is unchanged).
template <bool RESIDENT>
__global__ void __launch_bounds__(kWsThreads, 1)
proj_gemm_ws_kernel(const __grid_constant__ CUtensorMap mapA1, const __grid_constant__ CUtensorMap mapB1hi,
                    const __grid_constant__ CUtensorMap mapB1lo, const __grid_constant__ CUtensorMap mapA2,
                    const __grid_constant__ CUtensorMap mapB2hi, const __grid_constant__ CUtensorMap mapB2lo,
                    const __grid_constant__ CUtensorMap mapC, const ProjArgs p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) WsBars bars;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // streaming: stage s = {A, B-hi, B-lo} of one K-block; resident: B-hi/B-lo of K-block kb at the front,
    // then a ring of A blocks
    auto stage_ptr = [&](int s, int which) -> float* {
        if constexpr (RESIDENT) return reinterpret_cast<float*>(base + (2 * kResidentKb + s) * kTileBytes);
        else return reinterpret_cast<float*>(base + s * kStageBytes + which * kTileBytes);
    };
    auto resident_b = [&](int kb, int which) -> float* { return reinterpret_cast<float*>(base + (2 * kb + which) * kTileBytes); };
    float* patches = reinterpret_cast<float*>(base + kStages * kStageBytes);

    const long long n_tiles = (p.N + kBN - 1) / kBN, m_tiles = (p.M + kBM - 1) / kBM;
    const long long tiles = n_tiles * m_tiles;
    const int nkb = p.kb1 + p.kb2;
    // the tiles of this CTA: streaming deals all tiles round-robin; resident keeps the column tile and
    // strides over the row tiles (the grid is a multiple of n_tiles)
    const long long t_begin = RESIDENT ? blockIdx.x / n_tiles : blockIdx.x;
    const long long t_step = RESIDENT ? gridDim.x / n_tiles : gridDim.x;
    const long long t_end = RESIDENT ? m_tiles : tiles;
    const long long my_n = blockIdx.x % n_tiles;
    auto decode = [&](long long t, long long& m_tile, long long& n_tile) {
        if constexpr (RESIDENT) m_tile = t, n_tile = my_n;
        else m_tile = t / n_tiles, n_tile = t - m_tile * n_tiles;
    };

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars.full[s], 1);
            mbar_init(&bars.ready[s], 128);
            mbar_init(&bars.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars.acc_full[b], 1);
            mbar_init(&bars.acc_empty[b], 128);
        }
        mbar_init(&bars.b_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;
    const uint32_t tmem_a = tmem_d + (uint32_t)kTmemAcc;  // A ring: stage s at columns s*64 (hi) and s*64+32 (lo)

    // a bounded wait that also gives up when another role has raised the abort flag
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        const uint32_t a = smem_u32(bar);
        for (int i = 0; i < kWaitLimit; ++i) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(a), "r"(parity)
                : "memory");
            if (ok) return true;
            if (abort_flag) return false;
            __nanosleep(32);
        }
        abort_flag = 1;
        return false;
    };

    if (wid == 8) {
        // ------------------------------------------------------------ producer (one lane)
        if (lane == 0) {
            long long it = 0;
            if (RESIDENT && t_begin < t_end) {  // the column tile's split weights, once
                mbar_expect_tx(&bars.b_full, 2 * nkb * kTileBytes);
                for (int kb = 0; kb < nkb; ++kb) {
                    tma_load_2d(resident_b(kb, 0), &mapB1hi, kb * kBK, (int)(my_n * kBN), &bars.b_full);
                    tma_load_2d(resident_b(kb, 1), &mapB1lo, kb * kBK, (int)(my_n * kBN), &bars.b_full);
                }
            }
            for (long long t = t_begin; t < t_end && !abort_flag; t += t_step) {
                long long m_tile, n_tile;
                decode(t, m_tile, n_tile);
                const int row0 = (int)(m_tile * kBM), col0 = (int)(n_tile * kBN);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % kStages);
                    const uint32_t ph = (uint32_t)((it / kStages) & 1);
                    if (!wait(&bars.empty[s], ph ^ 1u)) break;  // a fresh barrier passes the wait for the phase before its first
                    const bool first = kb < p.kb1;
                    const int kx = (first ? kb : kb - p.kb1) * kBK;
                    mbar_expect_tx(&bars.full[s], (RESIDENT ? 1 : 3) * kTileBytes);
                    tma_load_2d(stage_ptr(s, 0), first ? &mapA1 : &mapA2, kx, row0, &bars.full[s]);
                    if constexpr (!RESIDENT) {
                        tma_load_2d(stage_ptr(s, 1), first ? &mapB1hi : &mapB2hi, kx, col0, &bars.full[s]);
                        tma_load_2d(stage_ptr(s, 2), first ? &mapB1lo : &mapB2lo, kx, col0, &bars.full[s]);
                    }
                }
            }
        }
    } else if (wid == 9) {
        // ------------------------------------------------------------ MMA issuer (one lane)
        if (lane == 0) {
            long long it = 0, ti = 0;
            if (RESIDENT && t_begin < t_end && !wait(&bars.b_full, 0)) abort_flag = 1;
            for (long long t = t_begin; t < t_end && !abort_flag; t += t_step, ++ti) {
                const int buf = (int)(ti & 1);
                if (!wait(&bars.acc_empty[buf], (uint32_t)(((ti >> 1) & 1) ^ 1))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_d + (uint32_t)(buf * kBN);
                bool fine = true;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = (int)(it % kStages);
                    if (!wait(&bars.ready[s], (uint32_t)((it / kStages) & 1))) {
                        fine = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t aHi = tmem_a + (uint32_t)(s * 64), aLo = aHi + 32u;
                    const uint64_t dBh = umma_desc_k_sw128(smem_u32(RESIDENT ? resident_b(kb, 0) : stage_ptr(s, 1)));
                    const uint64_t dBl = umma_desc_k_sw128(smem_u32(RESIDENT ? resident_b(kb, 1) : stage_ptr(s, 2)));
#pragma unroll
                    for (int k = 0; k < kBK / 8; ++k) {  // 8 TF32 per MMA along K: 8 columns of A, 32 bytes of B
                        const uint64_t adv = (uint64_t)(2 * k);
                        umma_tf32_ts(acc, aLo + (uint32_t)(8 * k), dBh + adv, (kb | k) != 0);
                        umma_tf32_ts(acc, aHi + (uint32_t)(8 * k), dBl + adv, 1u);
                        umma_tf32_ts(acc, aHi + (uint32_t)(8 * k), dBh + adv, 1u);
                    }
                    umma_commit(&bars.empty[s]);  // the stage (shared and tensor memory) is free once these MMAs have read it
                }
                if (!fine) break;
                umma_commit(&bars.acc_full[buf]);  // ... and the tile is complete once they have all finished
            }
        }
    } else if (wid >= 4) {
        // ------------------------------------------------------------ splitters (warps 4-7: lane quarter wid-4)
        const int row = (wid - 4) * 32 + lane;  // this thread's row of the block = its tensor-memory lane
        const uint32_t lane_field = (uint32_t)((wid - 4) * 32) << 16;
        long long it = 0;
        for (long long t = t_begin; t < t_end && !abort_flag; t += t_step) {
            bool fine = true;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = (int)(it % kStages);
                if (!wait(&bars.full[s], (uint32_t)((it / kStages) & 1))) {
                    fine = false;
                    break;
                }
                // row `row` of the 128-byte-swizzled block: its j-th 16-byte piece sits at piece j ^ (row % 8)
                const float4* arow = reinterpret_cast<const float4*>(stage_ptr(s, 0)) + row * 8;
                const uint32_t dst = tmem_a + lane_field + (uint32_t)(s * 64);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 x = arow[(half * 4 + j) ^ (row & 7)];
                        split_tf32(x.x, hi[4 * j], lo[4 * j]), split_tf32(x.y, hi[4 * j + 1], lo[4 * j + 1]);
                        split_tf32(x.z, hi[4 * j + 2], lo[4 * j + 2]), split_tf32(x.w, hi[4 * j + 3], lo[4 * j + 3]);
                    }
                    tmem_st16(dst + (uint32_t)(half * 16), hi);
                    tmem_st16(dst + 32u + (uint32_t)(half * 16), lo);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars.ready[s])) : "memory");
            }
            if (!fine) break;
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 0-3)
        float* patch = patches + wid * (2 * 32 * 32);  // this warp's two patches (the plain path uses them as one, pitch 36)
        long long ti = 0, pc = 0;                        // tiles and patches done
        for (long long t = t_begin; t < t_end && !abort_flag; t += t_step, ++ti) {
            long long m_tile, n_tile;
            decode(t, m_tile, n_tile);
            const long long row0 = m_tile * kBM, col0 = n_tile * kBN;
            const int buf = (int)(ti & 1);
            if (!wait(&bars.acc_full[buf], (uint32_t)((ti >> 1) & 1))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_d + (uint32_t)(buf * kBN) + ((uint32_t)(wid * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                float v[32];
                tmem_ld32(acc + (uint32_t)(c * 32), v);
                if (c == kBN / 32 - 1) {  // the accumulator is in registers: hand it back before storing
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars.acc_empty[buf])) : "memory");
                }
                const long long gc0 = col0 + c * 32;
                if (p.tma_c) {
                    if (gc0 >= p.N) continue;  // a column chunk past the end (uniform over the warp)
                    if (p.bias != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (gc0 + j < p.N) v[j] += __ldg(p.bias + gc0 + j);
                    }
                    float* pt = patch + (int)(pc & 1) * (32 * 32);
                    if (lane == 0) bulk_wait_read<1>();  // the store that read this patch two patches ago is done with it
                    __syncwarp();
                    // row `lane` of the patch: its q-th 16-byte piece sits at piece q ^ (lane % 8)
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(pt + lane * 32 + ((q ^ (lane & 7)) << 2)) =
                            make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> visible to the TMA unit
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&mapC, pt, (int)gc0, (int)(row0 + wid * 32));
                        bulk_commit();
                    }
                    ++pc;  // one group per patch: the patches alternate exactly with the groups
                    continue;
                }
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    *reinterpret_cast<float4*>(patch + lane * 36 + q * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                __syncwarp();
                const int cc = (lane & 7) * 4;
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int r = rr * 4 + (lane >> 3);
                    const long long grow = row0 + wid * 32 + r, gcol = gc0 + cc;
                    if (grow < p.M && gcol < p.N) {
                        float4 o = *reinterpret_cast<const float4*>(patch + r * 36 + cc);
                        if (p.bias != nullptr) {
                            o.x += p.bias[gcol];
                            if (gcol + 1 < p.N) o.y += p.bias[gcol + 1];
                            if (gcol + 2 < p.N) o.z += p.bias[gcol + 2];
                            if (gcol + 3 < p.N) o.w += p.bias[gcol + 3];
                        }
                        float* dst = p.C + grow * p.ldc + gcol;
                        if (gcol + 3 < p.N) {
                            __stcs(reinterpret_cast<float4*>(dst), o);
                        } else {
                            const float ov[4] = {o.x, o.y, o.z, o.w};
                            for (int e = 0; e < 4 && gcol + e < p.N; ++e) dst[e] = ov[e];
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (lane == 0) bulk_wait_all();  // this warp's stores have left shared memory and are complete
    }
    __syncwarp();  // the single-lane roles rejoin their warps before the CTA-wide barrier below
    // wind down together; copies a producer has in flight get a bounded time to land before the CTA's
    // shared memory is given up
    if (abort_flag && tid == 0) {
        atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTmemCols) : "memory");
    }
}

// ================================================================================ weight gradient
// dW[N, K] = G[M, N]^T * A[M, K]: the reduction runs over the tokens (rows of both operands), which are
// the slow axis in memory.  The activations A reach the tensor core "MN-major" from shared memory: a
// block of kTok tokens x 32 columns lands as kTok rows of 128 bytes, swizzled in 32-byte chunks with a
// period of 4 rows (the layout the tensor core expects of MN-major 4-byte elements), and the descriptor
// names the column axis as the contiguous one (leading byte offset = distance between two 32-column
// blocks, stride byte offset = 4 tokens = 512 bytes).  The output gradient G goes through tensor memory
// (below).  An MMA consumes 8 tokens; a CTA owns one 128 x 128 tile of dW for one slice of the token
// axis, accumulates it in tensor memory over its whole slice and writes it to the workspace;
// wgrad_reduce_kernel adds the slices in a fixed order.
constexpr int kTok = 32;                         // tokens per block
constexpr int kColBlk = kTok * 128;              // bytes of one 32-column block: kTok rows of 128 bytes

__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)(kColBlk >> 4) << 16;  // leading byte offset: next 32-column block
    d |= (uint64_t)(512 >> 4) << 32;      // stride byte offset: next group of 4 tokens (the swizzle period)
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;               // 128-byte swizzle with a 32-byte base (4-byte elements, MN-major)
    return d;
}
struct WgradArgs {
    float* part;        // [splits][N][Kp] partial sums
    long long M, N, K, Kp;
    long long tok_per_split;  // multiple of kTok
    int n_tiles, k_tiles;
    WsHeader* hdr;
};

// The phases of consecutive token blocks overlap and the G operand lives in tensor memory.  288 threads:
// warps 0-3 split G, warps 4-7 split A, lane 0 of warp 8 asks for the copies and issues the MMAs.  Per
// stage (two of them): the TMA unit brings the raw G block [32 tokens x 128 columns] (unswizzled: thread
// f reads column f down the tokens, conflict-free) and the A block (token-major, 32-byte-atom swizzle);
// the G splitters write hi and lo halves into tensor memory - feature f is lane f, the 32 tokens are 32
// columns - from where the MMAs take them as their A operand; the A splitters split the activation
// block in place (hi) and beside it (lo); the issuer launches the 12 MMAs (A from tensor memory, B = the
// activations, MN-major from shared memory), waits for them and asks for the block after next into
// the same stage while the splitters are busy with the other stage.  G never goes back to shared memory
// and is never read from there by the tensor core (a third less shared-memory traffic per block than
// splitting both operands there), and copy, split and MMA of neighbouring blocks run at the same time.
constexpr int kWgStages = 2;
constexpr int kWgStageBytes = 3 * kTileBytes;  // raw G, A (hi in place), A lo
constexpr int kWgSmem = kWgStages * kWgStageBytes + 1024;
constexpr int kWgThreads = 288;  // warps 0-3 split G, warps 4-7 split A, warp 8 copies and issues
constexpr uint32_t kIdescTsMN = kIdesc | (1u << 16);  // A from tensor memory, B MN-major

__device__ __forceinline__ void umma_tf32_ts_mn(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(kIdescTsMN), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(kWgThreads, 2)
proj_wgrad_ws_kernel(const __grid_constant__ CUtensorMap mapGraw, const __grid_constant__ CUtensorMap mapA, const WgradArgs p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[kWgStages], ready[kWgStages], done[kWgStages];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    auto sG = [&](int s) { return reinterpret_cast<float*>(base + s * kWgStageBytes); };
    auto sA = [&](int s) { return reinterpret_cast<float*>(base + s * kWgStageBytes + kTileBytes); };
    auto sAlo = [&](int s) { return reinterpret_cast<float*>(base + s * kWgStageBytes + 2 * kTileBytes); };

    const int tiles = p.n_tiles * p.k_tiles;
    const int split = blockIdx.x / tiles, t = blockIdx.x - split * tiles;
    const int n_tile = t / p.k_tiles, k_tile = t - n_tile * p.k_tiles;
    const int n0 = n_tile * 128, k0 = k_tile * 128;
    const long long tok0 = (long long)split * p.tok_per_split;
    long long tok1 = tok0 + p.tok_per_split;
    if (tok1 > p.M) tok1 = p.M;
    const int nblk = tok1 > tok0 ? (int)((tok1 - tok0 + kTok - 1) / kTok) : 0;

    if (tid == 0) {
        for (int s = 0; s < kWgStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&ready[s], 256);
            mbar_init(&done[s], 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(256)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;          // accumulator: columns [0, 128)
    const uint32_t tmem_g = tmem_d + 128u;           // G operand: stage s at columns 128 + 64 s (hi) and + 32 (lo)

    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        const uint32_t a = smem_u32(bar);
        for (int i = 0; i < kWaitLimit; ++i) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(a), "r"(parity)
                : "memory");
            if (ok) return true;
            if (abort_flag) return false;
            __nanosleep(32);
        }
        abort_flag = 1;
        return false;
    };

    if (wid == 8) {
        // ------------------------------------------------------------ copies and MMAs (one lane)
        if (lane == 0) {
            // rows past the slice's end but inside M belong to the next slice: slices are whole multiples of
            // kTok, so only the last one meets the end of the matrix (where the tensor maps fill zeros)
            auto request = [&](int kb) {
                const int s = kb % kWgStages;
                const int row = (int)(tok0 + (long long)kb * kTok);
                mbar_expect_tx(&full[s], 2 * kTileBytes);
                tma_load_2d(sG(s), &mapGraw, n0, row, &full[s]);
#pragma unroll
                for (int cb = 0; cb < 4; ++cb)
                    tma_load_2d(reinterpret_cast<unsigned char*>(sA(s)) + cb * kColBlk, &mapA, k0 + cb * 32, row, &full[s]);
            };
            for (int kb = 0; kb < kWgStages && kb < nblk; ++kb) request(kb);
            for (int kb = 0; kb < nblk && !abort_flag; ++kb) {
                const int s = kb % kWgStages;
                const uint32_t ph = (uint32_t)((kb / kWgStages) & 1);
                if (!wait(&ready[s], ph)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t gHi = tmem_g + (uint32_t)(s * 64), gLo = gHi + 32u;
                const uint64_t dA = umma_desc_mn_sw128(smem_u32(sA(s))), dAl = umma_desc_mn_sw128(smem_u32(sAlo(s)));
#pragma unroll
                for (int g = 0; g < kTok / 8; ++g) {  // 8 tokens per MMA: 8 columns of G, the next 1024-byte group of A
                    const uint64_t adv = (uint64_t)(g * (1024 >> 4));
                    umma_tf32_ts_mn(tmem_d, gLo + (uint32_t)(8 * g), dA + adv, (kb | g) != 0);
                    umma_tf32_ts_mn(tmem_d, gHi + (uint32_t)(8 * g), dAl + adv, 1u);
                    umma_tf32_ts_mn(tmem_d, gHi + (uint32_t)(8 * g), dA + adv, 1u);
                }
                umma_commit(&done[s]);
                // the stage (shared and tensor memory) is free once these MMAs have read it; the other stage
                // is being split meanwhile
                if (kb + kWgStages < nblk) {
                    if (!wait(&done[s], ph)) break;
                    request(kb + kWgStages);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ splitters (warps 0-3: G, 4-7: A); warps 0-3 then the epilogue
        const uint32_t lane_field = (uint32_t)((wid & 3) * 32) << 16;
        const bool g_side = wid < 4;
        const int st = tid & 127;  // index among the 128 threads of this side
        bool fine = true;
        for (int kb = 0; kb < nblk && !abort_flag; ++kb) {
            const int s = kb % kWgStages;
            if (!wait(&full[s], (uint32_t)((kb / kWgStages) & 1))) {
                fine = false;
                break;
            }
            if (g_side) {
                // G: column st of the block, token by token -> lane st of tensor memory, 32 columns hi, 32 lo
                const float* gcol = sG(s) + st;
                const uint32_t dst = tmem_g + lane_field + (uint32_t)(s * 64);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) split_tf32(gcol[(half * 16 + j) * 128], hi[j], lo[j]);
                    tmem_st16(dst + (uint32_t)(half * 16), hi);
                    tmem_st16(dst + 32u + (uint32_t)(half * 16), lo);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            } else {
                // A: hi in place, lo beside it (same swizzled position)
                float4* a4 = reinterpret_cast<float4*>(sA(s));
                float4* l4 = reinterpret_cast<float4*>(sAlo(s));
#pragma unroll
                for (int j = 0; j < kTileBytes / 16 / 128; ++j) {
                    const float4 y = a4[j * 128 + st];
                    float4 h, l;
                    split_tf32(y.x, h.x, l.x), split_tf32(y.y, h.y, l.y), split_tf32(y.z, h.z, l.z), split_tf32(y.w, h.w, l.w);
                    a4[j * 128 + st] = h;
                    l4[j * 128 + st] = l;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ready[s])) : "memory");
        }
        // all MMAs have finished once the last block's have (they complete in order)
        if (g_side && fine && nblk > 0 && !wait(&done[(nblk - 1) % kWgStages], (uint32_t)(((nblk - 1) / kWgStages) & 1))) fine = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (g_side && fine && !abort_flag) {
            // accumulator lane = row of dW (column of G), accumulator column = column of dW (column of A)
            float* patch = reinterpret_cast<float*>(base) + wid * (32 * 36);
            float* dst_tile = p.part + (long long)split * p.N * p.Kp;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float v[32];
                if (nblk > 0) {
                    tmem_ld32(tmem_d + lane_field + (uint32_t)(c * 32), v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    *reinterpret_cast<float4*>(patch + lane * 36 + q * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                __syncwarp();
                const int cc = (lane & 7) * 4;
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const int r = rr * 4 + (lane >> 3);
                    const long long grow = (long long)n0 + wid * 32 + r, gcol2 = (long long)k0 + c * 32 + cc;
                    if (grow < p.N && gcol2 < p.Kp)  // Kp is a multiple of 4: whole float4 pieces
                        *reinterpret_cast<float4*>(dst_tile + grow * p.Kp + gcol2) = *reinterpret_cast<const float4*>(patch + r * 36 + cc);
                }
                __syncwarp();
            }
        }
    }
    __syncwarp();
    if (abort_flag && tid == 0) {
        atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // give copies still in flight a bounded time to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(256) : "memory");
    }
}

// dW[n][k] = sum over slices of part[s][n][k] in a fixed order (reproducible)
__global__ void wgrad_reduce_kernel(const float* __restrict__ part, int splits, long long N, long long K, long long Kp,
                                    float* __restrict__ dW, long long lddw) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * K) return;
    const long long n = i / K, k = i - n * K;
    // eight running sums (slice sp goes to sum sp % 8) so that many loads are in flight; the sums are
    // then added in a fixed tree
    const float* src = part + n * Kp + k;
    const long long stride = N * Kp;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int sp = 0;
#pragma unroll 2
    for (; sp + 8 <= splits; sp += 8) {
#pragma unroll
        for (int r = 0; r < 8; ++r) acc[r] += src[(long long)(sp + r) * stride];
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
        if (sp + r < splits) acc[r] += src[(long long)(sp + r) * stride];
    dW[n * lddw + k] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Tensor map of a row-major float32 matrix [rows, cols] (row pitch ld floats) read in boxes of
// box_cols (kBK unless stated) columns x box_rows rows into the named shared-memory layout; rows and columns
// past the end read as zero.
static bool make_map(CUtensorMap* map, const float* ptr, long long rows, long long cols, long long ld, int box_rows = kBM,
                     CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, int box_cols = kBK) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct ProjWs {
    size_t off_b1hi, off_b1lo, off_b2hi, off_b2lo, total;
};
static long long pad4(long long k) { return (k + 3) / 4 * 4; }
static ProjWs proj_ws(long long N, long long K1, long long K2) {
    ProjWs w;
    size_t off = align_up(sizeof(WsHeader), 256);
    const size_t s1 = align_up(sizeof(float) * (size_t)(N * pad4(K1)), 256), s2 = align_up(sizeof(float) * (size_t)(N * pad4(K2)), 256);
    w.off_b1hi = off, off += s1;
    w.off_b1lo = off, off += s1;
    w.off_b2hi = off, off += s2;
    w.off_b2lo = off, off += s2;
    w.total = off;
    return w;
}


// Token slices of the weight gradient: enough CTAs to fill every SM (two per SM: each holds 256 of the
// 512 tensor-memory columns), slices a multiple of kTok.
constexpr int kWgradCtasPerSm = 2;
struct WgradPlan {
    int n_tiles, k_tiles, splits;
    long long tok_per_split, Kp;
    size_t off_part, total;
};
static WgradPlan wgrad_plan(long long M, long long N, long long K) {
    WgradPlan w;
    w.n_tiles = (int)((N + 127) / 128), w.k_tiles = (int)((K + 127) / 128);
    w.Kp = pad4(K);
    const long long tiles = (long long)w.n_tiles * w.k_tiles;
    long long want = (kWgradCtasPerSm * 148 + tiles - 1) / tiles;  // slices so that every SM has its resident CTAs
    const long long blocks = (M + kTok - 1) / kTok;
    if (want > blocks) want = blocks;
    if (want < 1) want = 1;
    const long long bps = (blocks + want - 1) / want;  // token blocks per slice
    w.tok_per_split = bps * kTok;
    w.splits = (int)((blocks + bps - 1) / bps);
    w.off_part = align_up(sizeof(WsHeader), 256);
    w.total = w.off_part + align_up(sizeof(float) * (size_t)w.splits * (size_t)N * (size_t)w.Kp, 256);
    return w;
}

static int sm_count_proj() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static bool row_ok(const void* p, long long ld) { return p != nullptr && ((uintptr_t)p & 15) == 0 && ld % 4 == 0; }

}  // namespace b200

extern "C" {

size_t b200_proj_gemm_workspace_bytes(int64_t N, int64_t K1, int64_t K2) {
    if (N <= 0 || K1 < 0 || K2 < 0) return 256;
    return b200::proj_ws(N, K1, K2).total;
}

int b200_proj_gemm(int64_t M, int64_t N, int64_t K1, const void* A1, int64_t lda1, const void* B1, int64_t ldb1,
                   int64_t K2, const void* A2, int64_t lda2, const void* B2, int64_t ldb2, const void* bias, void* C,
                   int64_t ldc, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace b200;
    if (M < 0 || N <= 0 || K1 <= 0 || K2 < 0) return B200_ERR_ARG;
    if (M == 0) return B200_OK;
    if (!row_ok(A1, lda1) || !B1 || !C || ldc < N || lda1 < K1 || ldb1 < K1) return B200_ERR_ARG;
    if (K2 > 0 && (!row_ok(A2, lda2) || !B2 || lda2 < K2 || ldb2 < K2)) return B200_ERR_ARG;
    if (((uintptr_t)C & 15) != 0 || ldc % 4 != 0) return B200_ERR_ARG;
    const ProjWs w = proj_ws(N, K1, K2);
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < w.total) return B200_ERR_WORKSPACE;
    const long long tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    if (tiles > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* base = static_cast<char*>(workspace);
    if (cudaMemsetAsync(base, 0, sizeof(WsHeader), st) != cudaSuccess) return B200_ERR_LAUNCH;
    float* b1hi = (float*)(base + w.off_b1hi);
    float* b1lo = (float*)(base + w.off_b1lo);
    float* b2hi = (float*)(base + w.off_b2hi);
    float* b2lo = (float*)(base + w.off_b2lo);
    const long long K1p = pad4(K1), K2p = pad4(K2);
    split_weights_kernel<<<(unsigned int)((N * K1p + 255) / 256), 256, 0, st>>>((const float*)B1, ldb1, N, K1, K1p, b1hi, b1lo);
    if (K2 > 0)
        split_weights_kernel<<<(unsigned int)((N * K2p + 255) / 256), 256, 0, st>>>((const float*)B2, ldb2, N, K2, K2p, b2hi, b2lo);
    if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;

    CUtensorMap mA1, mB1h, mB1l, mA2, mB2h, mB2l;
    bool ok = make_map(&mA1, (const float*)A1, M, K1, lda1) && make_map(&mB1h, b1hi, N, K1, K1p) && make_map(&mB1l, b1lo, N, K1, K1p);
    if (K2 > 0) {
        ok = ok && make_map(&mA2, (const float*)A2, M, K2, lda2) && make_map(&mB2h, b2hi, N, K2, K2p) && make_map(&mB2l, b2lo, N, K2, K2p);
    } else {
        mA2 = mA1, mB2h = mB1h, mB2l = mB1l;
    }
    if (!ok) return B200_ERR_LAUNCH;

    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(proj_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess ||
            cudaFuncSetAttribute(proj_gemm_ws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmem) != cudaSuccess ||
            cudaFuncSetAttribute(proj_gemm_ws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    ProjArgs a;
    a.C = (float*)C, a.bias = (const float*)bias, a.ldc = ldc, a.M = M, a.N = N;
    // C through TMA when its rows are 16-byte aligned (32 x 32 boxes, 128-byte swizzle in shared memory)
    CUtensorMap mC = mA1;
    a.tma_c = (PROJ_TMA_STORE && row_ok(C, ldc) && make_map(&mC, (const float*)C, M, N, ldc, 32)) ? 1 : 0;
    a.kb1 = (int)((K1 + kBK - 1) / kBK), a.kb2 = (int)((K2 + kBK - 1) / kBK);  // a ragged last block reads zeros past K
    a.hdr = reinterpret_cast<WsHeader*>(base);
#ifdef PROJ_GEMM_SIMPLE
    proj_gemm_kernel<<<(unsigned int)tiles, 128, kGemmSmem, st>>>(mA1, mB1h, mB1l, mA2, mB2h, mB2l, a);
#else
    // few tiles: the one-tile-per-CTA kernel spreads them over more SMs than one persistent CTA per SM could
    const long long sms = sm_count_proj(), n_tiles = (N + kBN - 1) / kBN;
    if (tiles < 2 * sms) {
        proj_gemm_kernel<<<(unsigned int)tiles, 128, kGemmSmem, st>>>(mA1, mB1h, mB1l, mA2, mB2h, mB2l, a);
    } else if (PROJ_RESIDENT && a.kb2 == 0 && a.kb1 <= kResidentKb && n_tiles <= sms) {
        // short K: the column tile's weights stay in shared memory; whole groups of n_tiles CTAs
        const long long grid = sms - sms % n_tiles;
        proj_gemm_ws_kernel<true><<<(unsigned int)grid, kWsThreads, kWsSmem, st>>>(mA1, mB1h, mB1l, mA2, mB2h, mB2l, mC, a);
    } else {
        proj_gemm_ws_kernel<false><<<(unsigned int)sms, kWsThreads, kWsSmem, st>>>(mA1, mB1h, mB1l, mA2, mB2h, mB2l, mC, a);
    }
#endif
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

size_t b200_proj_wgrad_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 256;
    return b200::wgrad_plan(M, N, K).total;
}

int b200_proj_wgrad(int64_t M, int64_t N, int64_t K, const void* G, int64_t ldg, const void* A, int64_t lda, void* dW,
                    int64_t lddw, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace b200;
    if (M < 0 || N <= 0 || K <= 0 || !dW || lddw < K) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M == 0) {
        if (cudaMemset2DAsync(dW, (size_t)lddw * 4, 0, (size_t)K * 4, (size_t)N, st) != cudaSuccess) return B200_ERR_LAUNCH;
        return B200_OK;
    }
    if (!row_ok(G, ldg) || !row_ok(A, lda) || ldg < N || lda < K) return B200_ERR_ARG;
    const WgradPlan w = wgrad_plan(M, N, K);
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < w.total) return B200_ERR_WORKSPACE;
    char* base = static_cast<char*>(workspace);
    if (cudaMemsetAsync(base, 0, sizeof(WsHeader), st) != cudaSuccess) return B200_ERR_LAUNCH;
    CUtensorMap mG, mA;
    // G as plain rows of 128 columns (threads read it, not the tensor core); the token-major activations of
    // 4-byte elements in the 128-byte swizzle whose unit is a 32-byte chunk
    if (!make_map(&mG, (const float*)G, M, N, ldg, kTok, CU_TENSOR_MAP_SWIZZLE_NONE, 128) ||
        !make_map(&mA, (const float*)A, M, K, lda, kTok, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
        return B200_ERR_LAUNCH;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(proj_wgrad_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    WgradArgs a;
    a.part = (float*)(base + w.off_part);
    a.M = M, a.N = N, a.K = K, a.Kp = w.Kp, a.tok_per_split = w.tok_per_split;
    a.n_tiles = w.n_tiles, a.k_tiles = w.k_tiles;
    a.hdr = reinterpret_cast<WsHeader*>(base);
    const long long grid = (long long)w.splits * w.n_tiles * w.k_tiles;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    proj_wgrad_ws_kernel<<<(unsigned int)grid, kWgThreads, kWgSmem, st>>>(mG, mA, a);
    if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;
    wgrad_reduce_kernel<<<(unsigned int)((N * K + 255) / 256), 256, 0, st>>>(a.part, w.splits, N, K, w.Kp, (float*)dW, lddw);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
