// All-reduce of small row-parallel outputs over NVLink peer memory.
//
// The decode step of a tensor-parallel model sums a [M, hidden] tile (tens of KB)
// across ranks after every row-parallel linear.  At that size a library
// collective is pure latency (protocol set-up, several kernel phases), so this
// file has a one-shot kernel instead:
//
//   * every rank owns one region (cudaMalloc) that all other ranks of the node map
//     through CUDA IPC: data[2 phases][rank][slot] plus arrival flags;
//   * push: a CTA copies its slice of the local tile into slot `my rank` of EVERY
//     rank's region (plain 16-byte stores, remote ones travel over NVLink), then
//     one thread per peer publishes the call's epoch with st.release.sys;
//   * wait: the CTA polls ITS OWN region's flags (ld.acquire.sys) until every rank's
//     epoch arrived - bounded; on expiry it raises an error word and leaves;
//   * reduce: sums the slots in rank order in fp32 and writes the tile back.
//     Every rank adds the same numbers in the same order: results are bit-identical
//     on all ranks and from run to run.
//
// Two phases (epoch parity) are enough: a rank can be at most one call ahead of the
// slowest rank, because finishing call k needs every peer's data of call k, and a
// rank's calls run one after another on its stream.
//
// Plain peer stores and local loads only (no bulk-copy engine, no switch reductions).
#include "gaf_internal.h"

#include <cuda_bf16.h>

namespace tgaf {

namespace {

constexpr uint32_t kPeerWaitLimit = 1u << 23;  // polls with back-off (several seconds: ranks may start far apart) before giving up

struct PeerArgs {
    uint8_t *region[kPeerMaxRanks];  // every rank's region as mapped here; [rank] is the local one
    uint32_t rank, size;
    unsigned int *error_word;
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr size_t kFlagsOff = kPeerFlagsOff, kEpochOff = kPeerEpochOff, kDataOff = kPeerDataOff;
static_assert(2 * kPeerCtas * kPeerMaxRanks * 4 <= 4096, "flag block");

template <bool F32>
__device__ __forceinline__ void accumulate(float (&acc)[F32 ? 4 : 8], const uint4 &v) {
    if constexpr (F32) {
        acc[0] += __uint_as_float(v.x), acc[1] += __uint_as_float(v.y);
        acc[2] += __uint_as_float(v.z), acc[3] += __uint_as_float(v.w);
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] += __uint_as_float(w[i] << 16);
            acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
}

// buf: the tile as nvec 16-byte vectors (the host side only takes tiles that are a whole number of them).
template <bool F32>
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(const PeerArgs a, uint4 *buf, uint32_t nvec) {
    __shared__ uint32_t s_epoch;
    __shared__ uint32_t s_abort;
    uint8_t *mine = a.region[a.rank];
    const uint32_t cta = blockIdx.x, tid = threadIdx.x;
    // Only meaningful when launched with programmatic stream serialization (off by default: measured slower
    // than plain stream order on the decode stack): lets the next kernel start, then waits for the previous.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
        uint32_t *ep = reinterpret_cast<uint32_t *>(mine + kEpochOff) + cta;
        s_epoch = *ep + 1u;
        *ep = s_epoch;
        s_abort = 0u;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch, phase = epoch & 1u;
    const uint32_t per = (nvec + gridDim.x - 1u) / gridDim.x;
    const uint32_t lo = cta * per;
    const uint32_t hi = lo + per < nvec ? lo + per : nvec;
    if (lo >= hi) return;  // nothing in this CTA's slice (its epoch still advanced, like everybody's)

    // ---- push my slice into slot `rank` of every region ----
    const size_t slot_off = kDataOff + (static_cast<size_t>(phase) * kPeerMaxRanks + a.rank) * kPeerSlotBytes;
    for (uint32_t v = lo + tid; v < hi; v += blockDim.x) {
        const uint4 val = buf[v];
#pragma unroll
        for (uint32_t i = 0; i < kPeerMaxRanks; ++i) {
            if (i < a.size) {
                const uint32_t r = (a.rank + i) % a.size;  // start with myself, spread the peers
                reinterpret_cast<uint4 *>(a.region[r] + slot_off)[v] = val;
            }
        }
    }
    __syncthreads();
    if (tid < a.size) {
        uint32_t *flag = reinterpret_cast<uint32_t *>(a.region[tid] + kFlagsOff) + (phase * kPeerCtas + cta) * kPeerMaxRanks + a.rank;
        st_release_sys(flag, epoch);
    }

    // ---- wait for every rank's slice ----
    if (tid < a.size) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(mine + kFlagsOff) + (phase * kPeerCtas + cta) * kPeerMaxRanks + tid;
        bool ok = false;
        for (uint32_t it = 0; it < kPeerWaitLimit; ++it) {
            if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) {
                ok = true;
                break;
            }
            if (it > 64) __nanosleep(it > 4096 ? 1000 : 32);
        }
        if (!ok) {
            atomicOr(a.error_word, 0x100u);
            s_abort = 1u;
        }
    }
    __syncthreads();
    if (s_abort) return;

    // ---- add the slots in rank order ----
    const uint8_t *data = mine + kDataOff + static_cast<size_t>(phase) * kPeerMaxRanks * kPeerSlotBytes;
    for (uint32_t v = lo + tid; v < hi; v += blockDim.x) {
        float acc[F32 ? 4 : 8];
#pragma unroll
        for (int i = 0; i < (F32 ? 4 : 8); ++i) acc[i] = 0.f;
        uint4 in[kPeerMaxRanks];
#pragma unroll
        for (uint32_t r = 0; r < kPeerMaxRanks; ++r)
            if (r < a.size) in[r] = __ldcg(reinterpret_cast<const uint4 *>(data + r * kPeerSlotBytes) + v);
#pragma unroll
        for (uint32_t r = 0; r < kPeerMaxRanks; ++r)
            if (r < a.size) accumulate<F32>(acc, in[r]);
        uint4 out;
        if constexpr (F32) {
            out = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
        } else {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t *>(&p);
            }
            out = make_uint4(w[0], w[1], w[2], w[3]);
        }
        buf[v] = out;
    }
}

}  // namespace

size_t peer_region_bytes() { return kPeerRegionBytes; }

cudaError_t peer_allreduce(const PeerComm &pc, void *d_buf, size_t count, bool f32, bool pdl, cudaStream_t stream,
                           unsigned int *d_error_word) {
    const size_t bytes = count * (f32 ? 4u : 2u);
    if (!pc.ok || bytes == 0 || bytes > kPeerSlotBytes || bytes % 16u != 0 ||
        reinterpret_cast<uintptr_t>(d_buf) % 16u != 0)
        return cudaErrorNotSupported;
    PeerArgs a;
    for (int r = 0; r < kPeerMaxRanks; ++r) a.region[r] = static_cast<uint8_t *>(pc.region[r]);
    a.rank = pc.rank;
    a.size = pc.size;
    a.error_word = d_error_word;
    const uint32_t nvec = static_cast<uint32_t>(bytes / 16u);
    // always the full grid: every CTA's epoch advances on every call, on every rank
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kPeerCtas);
    cfg.blockDim = dim3(kPeerThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    uint4 *vbuf = static_cast<uint4 *>(d_buf);
    if (f32) return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<true>, a, vbuf, nvec);
    return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<false>, a, vbuf, nvec);
}

}  // namespace tgaf
