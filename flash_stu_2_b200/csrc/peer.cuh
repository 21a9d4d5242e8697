// Exchange of the token loop's sub-layer outputs between the GPUs of a tensor-parallel group, fused into the kernels
// that produce them: the producing kernel stores its result straight into every rank's inbox (plain stores to peer
// memory over NVLink) and, when its last CTA is done, raises one flag per rank; the consuming kernel waits (bounded)
// for the flags of all senders and reads its own inbox.  No load ever targets another GPU's memory.
#pragma once
#include "common.cuh"

#define STU_MAX_PEERS 8

// One exchange point (a fixed place in the token step) as a sender sees it; lives in the sender's device memory.
struct PeerDest {
  int n;                          // ranks (this one included)
  int pad;
  bf16* dest[STU_MAX_PEERS];      // where this rank's rows go inside rank p's inbox (slot and column offset applied)
  unsigned* flag[STU_MAX_PEERS];  // rank p's arrival counter for this sender
  unsigned* epoch;                // local: how many times this exchange has been sent
  unsigned* ctr;                  // local: CTAs of the running launch that have finished storing
};

// Called by ONE thread per CTA, after a CTA-wide barrier that follows the CTA's last store to the peers.  The last
// CTA of the launch to get here advances the local epoch and raises this sender's flag on every rank.
__device__ __forceinline__ void peer_signal_when_last(const PeerDest* pd, unsigned total_ctas) {
  __threadfence_system();
  const unsigned prev = atomicAdd(pd->ctr, 1u);
  if (prev == total_ctas - 1) {
    *pd->ctr = 0;   // for the next launch of this exchange
    atomicAdd(pd->epoch, 1u);
    __threadfence_system();
    for (int p = 0; p < pd->n; p++)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(pd->flag[p]) : "memory");
  }
}

// One exchange point as the exchange kernel (push + wait + combine in one launch, one CTA per row) sees it; lives in
// the device memory of the rank that runs the kernel.
struct PeerXchg {
  int n, rank;
  bf16* inbox[STU_MAX_PEERS];      // rank p's inbox of this exchange as mapped here: [slots][rows][d]
  unsigned* flag[STU_MAX_PEERS];   // rank p's arrival counters of this exchange: [n senders][rows]
  unsigned* epoch;                 // local [rows]: how many times each row has been exchanged
};
