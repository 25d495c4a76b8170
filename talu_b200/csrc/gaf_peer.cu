// All-reduce of small row-parallel outputs over NVLink peer memory.
//
// The decode step of a tensor-parallel model sums a [M, hidden] tile (tens of KB)
// across ranks after every row-parallel linear.  At that size a library
// collective is pure latency (protocol set-up, several kernel phases), so this
// file has a one-shot kernel instead:
//
//   * every rank owns one region (cudaMalloc) that all other ranks of the node map
//     through CUDA IPC: data[2 phases][rank][slot] plus per-CTA call counters;
//   * push: a CTA widens its slice of the local tile to fp32 and stores it into slot
//     `my rank` of EVERY rank's region as 64-bit words {fp32 value, call epoch}
//     (plain stores; the remote ones travel over NVLink).  One store carries value
//     and arrival: a reader that sees the epoch has the value - no flag, no fence,
//     one NVLink hop (the "LL" idea of collective libraries);
//   * wait + reduce: the CTA polls ITS OWN region for every rank's words of its slice
//     (bounded; on expiry it raises an error word and leaves), adds them in rank
//     order in fp32 and writes the tile back.  Every rank adds the same numbers in
//     the same order: results are bit-identical on all ranks and from run to run.
//
// Two phases (epoch parity) are enough: a rank can be at most one call ahead of the
// slowest rank, because finishing call k needs every peer's words of call k, and a
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
    uint32_t wait_size;   // ranks whose words are awaited (= size, or size + 1 for the diagnostic that makes a wait run out)
    uint32_t wait_limit;  // polls per awaited word
    unsigned int *error_word;
};

constexpr size_t kEpochOff = kPeerEpochOff, kDataOff = kPeerDataOff;

// buf: count elements (bf16 or f32); a slot holds count 64-bit words
template <bool F32>
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(const PeerArgs a, void *buf, uint32_t count) {
    __shared__ uint32_t s_epoch;
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
    }
    __syncthreads();
    const uint32_t epoch = s_epoch, phase = epoch & 1u;
    const uint32_t per = (count + gridDim.x - 1u) / gridDim.x;
    const uint32_t lo = cta * per;
    const uint32_t hi = lo + per < count ? lo + per : count;
    if (lo >= hi) return;  // nothing in this CTA's slice (its epoch still advanced, like everybody's)

    auto load_in = [&](uint32_t i) -> float {
        if constexpr (F32) return static_cast<const float *>(buf)[i];
        return __bfloat162float(static_cast<const __nv_bfloat16 *>(buf)[i]);
    };
    // ---- push my slice into slot `rank` of every region ----
    const size_t slot_off = kDataOff + (static_cast<size_t>(phase) * kPeerMaxRanks + a.rank) * kPeerSlotBytes;
    for (uint32_t i = lo + tid; i < hi; i += blockDim.x) {
        const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(load_in(i));
        for (uint32_t j = 0; j < a.size; ++j) {
            uint32_t r = a.rank + j;  // start with myself, spread the peers
            if (r >= a.size) r -= a.size;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long *>(a.region[r] + slot_off) + i), "l"(word)
                         : "memory");
        }
    }
    // ---- every rank's words of my slice, added in rank order ----
    const unsigned long long *data =
        reinterpret_cast<const unsigned long long *>(mine + kDataOff + static_cast<size_t>(phase) * kPeerMaxRanks * kPeerSlotBytes);
    for (uint32_t i = lo + tid; i < hi; i += blockDim.x) {
        float acc = 0.f;
        for (uint32_t r = 0; r < a.wait_size; ++r) {
            const unsigned long long *src = data + r * (kPeerSlotBytes / 8u) + i;
            unsigned long long word = 0ull;
            bool got = false;
            for (uint32_t it = 0; it < a.wait_limit; ++it) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
                if (static_cast<uint32_t>(word >> 32) == epoch) {
                    got = true;
                    break;
                }
                if (it > 64) __nanosleep(it > 4096 ? 1000 : 32);
            }
            if (!got) {
                atomicOr(a.error_word, 0x100u);
                return;  // no barrier follows: a thread may leave alone
            }
            acc += __uint_as_float(static_cast<uint32_t>(word));
        }
        if constexpr (F32)
            static_cast<float *>(buf)[i] = acc;
        else
            static_cast<__nv_bfloat16 *>(buf)[i] = __float2bfloat16_rn(acc);
    }
}

}  // namespace

size_t peer_region_bytes() { return kPeerRegionBytes; }

cudaError_t peer_allreduce(const PeerComm &pc, void *d_buf, size_t count, bool f32, bool pdl, cudaStream_t stream,
                           unsigned int *d_error_word, uint32_t wait_limit, bool expect_absent_rank) {
    // one 64-bit word per element in a slot
    if (!pc.ok || count == 0 || count * 8u > kPeerSlotBytes || reinterpret_cast<uintptr_t>(d_buf) % (f32 ? 4u : 2u) != 0)
        return cudaErrorNotSupported;
    PeerArgs a;
    for (int r = 0; r < kPeerMaxRanks; ++r) a.region[r] = static_cast<uint8_t *>(pc.region[r]);
    a.rank = pc.rank;
    a.size = pc.size;
    a.wait_size = pc.size + ((expect_absent_rank && pc.size < static_cast<uint32_t>(kPeerMaxRanks)) ? 1u : 0u);
    a.wait_limit = wait_limit ? wait_limit : kPeerWaitLimit;
    a.error_word = d_error_word;
    const uint32_t n = static_cast<uint32_t>(count);
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
    if (f32) return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<true>, a, d_buf, n);
    return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel<false>, a, d_buf, n);
}

}  // namespace tgaf
