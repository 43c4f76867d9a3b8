// Declarations shared by the library's own translation units (not part of the
// C-ABI): error reporting and the launch of one KV-sharded decode step, which
// shard.cc (host logic of the multi-GPU layer) calls and api.cu implements.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "tilefusion_b200.h"

namespace tfb {

// Records the text tf_last_error() returns on the calling thread; returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Per-device set-up that entry points share: the host-visible mirror of the
// device status word and the wait limit.  Returns a TfStatus.
int ensure_device_ready();

// One step of a KV-sharded decode.  All buffers belong to the TfShardCtx.
struct ShardStep {
  void* workspace;             // split-KV partial rows of this rank, then one flag word per (b, h, split):
  uint64_t workspace_bytes;    //   plan.workspace_bytes + batch*heads*num_splits*4 bytes; flag words start
                               //   at zero and hold the number of the last step that wrote their row
  unsigned* rows_done;         // one word, zero between steps
  float* const* peer_table;    // device array [n_ranks] of gather-buffer bases as mapped into this
                               // process; null = merged rows go to this rank's slot only (NCCL transport)
  float* local_base;           // this rank's gather buffer
  int n_ranks;
  int rank;
  long long area_offset;       // floats from a buffer base to the gather area of this step
  long long flag_offset;       // floats from a buffer base to the flag words
  unsigned step;
};

// Split pass with the merge fused in; with a peer table also the scatter to
// every rank's gather area, the flags, and the final combine into o / lse.
int launch_sharded_decode(const void* q, const void* k, const void* v, void* o, float* lse,
                          const TfDecodeDesc* desc, const ShardStep& step, cudaStream_t stream);

}  // namespace tfb
