// Layout of a rank's peer-mapped communication buffer and the flag accesses on it, shared by the
// stand-alone all-reduce kernel and the all-reduce epilogue of the streaming decode GEMM.
//
//   [0, 256)          status word (first int) of bounded waits; at byte 8 the wait limit in
//                     nanoseconds as a 64-bit integer (0: the default, one second)
//   [256, 512)        call counters of the stand-alone kernel, one per CTA (kArBlocks)
//   [512, 1536)       its flags: [CTA][source rank]
//   [4096, 20480)     flags of the GEMM epilogue: [flag set][source rank], kEpilogueSets sets
//   [20480, 22528)    call counters of the GEMM epilogue, one per flag set
//   [22528, 23040)    call counters of the two-shot kernel, one per CTA (kTsBlocks)
//   [23040, 27136)    its flags: [CTA][source rank]
//   [32768, ...)      data slots
#pragma once
#include <stdint.h>
#include <stddef.h>

namespace nqb200 {

constexpr int kMaxRanks = 8;
constexpr int kArBlocks = 32;
constexpr int kEpilogueSets = 512;
constexpr size_t kArOffWaitNs = 8;
constexpr unsigned long long kArDefaultWaitNs = 1000000000ull;
constexpr size_t kArOffEpoch = 256, kArOffFlags = 512;
constexpr size_t kArOffFlags2 = 4096, kArOffEpoch2 = kArOffFlags2 + (size_t)kEpilogueSets * kMaxRanks * 4;
constexpr int kTsBlocks = 128;
constexpr size_t kArOffEpoch3 = kArOffEpoch2 + (size_t)kEpilogueSets * 4, kArOffFlags3 = kArOffEpoch3 + (size_t)kTsBlocks * 4;
constexpr size_t kArOffData = 32768;
static_assert(kArOffFlags3 + (size_t)kTsBlocks * kMaxRanks * 4 <= kArOffData, "header overlaps the data slots");
static_assert(kArOffEpoch2 + (size_t)kEpilogueSets * 4 <= kArOffData, "header overlaps the data slots");

// What a GEMM needs to all-reduce its output over peer memory in its own epilogue.
struct PeerEpilogue {
  uint8_t* peers[kMaxRanks];  // every rank's buffer as mapped into this process (peers[rank] is our own)
  int rank, world;
  size_t slot_off;            // byte offset of the slot inside the data region
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_flag(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// the rank's wait limit (its own buffer's header; 0 means the default)
__device__ __forceinline__ unsigned long long peer_wait_limit_ns(const uint8_t* own) {
  const unsigned long long v = *reinterpret_cast<const unsigned long long*>(own + kArOffWaitNs);
  return v ? v : kArDefaultWaitNs;
}
__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
  uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
#endif

}  // namespace nqb200
