// Tensor-parallel exchange over NVLink peer memory: the layout of a rank's exchange block and the system-scope loads
// and stores every kernel that takes part in an exchange uses (tp_comm.cu: the stand-alone exchange kernels;
// gemv_w4a16.cu: the all-reduce inside the row-split GEMV).
#pragma once
#include "common.cuh"

namespace b200 {

// Layout of one rank's exchange block (allocated by comm_alloc, zeroed): a 256-byte header, then the data slots at
// offsets the caller chooses (multiples of 16 bytes).
constexpr int kCommHeaderBytes = 256;
constexpr int kCommMaxRanks = 16;
constexpr int kCommFlagsOff = 0;      // uint32 flags[16]: flags[j] = latest step rank j has announced to this rank
constexpr int kCommCounterOff = 64;   // uint32: steps this rank has taken
constexpr int kCommErrorOff = 68;     // uint32: 0, or the code of a wait that ran out
constexpr int kCommLimitOff = 72;     // uint32: polls before a wait for a peer gives up; 0 = kCommSpinLimit
constexpr int kCommThreads = 1024;
constexpr int kCommSpinLimit = 1 << 22;

enum : uint32_t { COMM_ERR_PEER_WAIT = 1 };

struct CommPeers {
  uint8_t* p[kCommMaxRanks];   // base of every rank's exchange block as mapped into this process; p[rank] is local
};

DEVI void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DEVI uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DEVI uint4 ld_peer16(const void* p) {
  uint4 r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p)
               : "memory");
  return r;
}

// ---- all-reduce inside a row-split GEMV (gemv_w4a16.cu: the ALLRED epilogue) ---------------------------------------
// A "GEMV slot" of the exchange block, at a caller-chosen offset (multiple of 256 bytes):
//   [0, 256)                       control: uint32 calls (exchanges completed on this slot), uint32 done (blocks of
//                                  the running call that have finished)
//   [256, 256 + 64 KB)             reserved (flag rows of an earlier form of the exchange)
//   [256 + 64 KB, ... + 16 N 4)    uint32 words[r][N] for r < W: rank r's partial rows as (tag << 16 | fp16), pushed
//                                  here by rank r; tag = low 16 bits of the call number + 1, never 0. A word that
//                                  carries the call's tag IS the arrival of its row: no flags, no fence, one NVLink
//                                  flight.
constexpr int kCommMaxGroups = 1024;
constexpr size_t kGemvSlotCtrlBytes = 256;
constexpr size_t kGemvSlotFlagBytes = (size_t)kCommMaxGroups * kCommMaxRanks * 4;
inline size_t gemv_slot_bytes(int N, int W) { return kGemvSlotCtrlBytes + kGemvSlotFlagBytes + (size_t)W * N * 4; }
DEVI uint32_t comm_tag(uint32_t call) { return ((call % 65535u) + 1u) << 16; }

struct AllReduceArgs {
  CommPeers P;
  int rank, W;     // W == 0: no exchange, the GEMV stores its rows to y
  size_t off;      // offset of the GEMV slot inside every rank's block
  int tagged;      // 1: push tagged words and return (no flags, no wait, no sum, y untouched)
};

DEVI void st_peer16(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace b200
