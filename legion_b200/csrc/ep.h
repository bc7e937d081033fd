// Launch interface of the expert-parallel dispatch kernels (ep.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define EP_MAX_RANKS 8
#define EP_SLOT_COUNTS 32
#define EP_SLOT_PUSHED 40
#define EP_SLOT_DONE 48

namespace lb {

struct EpPeers {
  void* buffer[EP_MAX_RANKS];   // peer-mapped base of every rank's symmetric EP buffer
  void* signal[EP_MAX_RANKS];   // peer-mapped signal pads (uint32 slots)
  int rank, world;
};

int ep_publish_counts_launch(const EpPeers& p, const int* counts, int E, long counts_off, const uint32_t* seq_ptr,
                             int* dest_base, int* recv_counts, int* meta, int cap, uint64_t budget_ns, int* status,
                             cudaStream_t s);
int ep_push_launch(const EpPeers& p, const void* x, long ldx, int H, const int* sorted_token, const int* sorted_pair,
                   const float* sorted_w, const int* offsets, const int* dest_base, int E, int cap, long rx_off,
                   long rsrc_off, long rw_off, const uint32_t* seq_ptr, unsigned int* done_ctr, int max_rows,
                   cudaStream_t s);
int ep_sync_launch(const EpPeers& p, int slot_base, int signal_first, uint32_t* seq_ptr, int bump, uint64_t budget_ns,
                   int* status, cudaStream_t s);
int moe_tiles_launch(const int* counts, int n_local, int bn, int* offsets, int* tile_group, int* tile_tok0,
                     int* tile_ntok, int max_tiles, int* meta, cudaStream_t s);

}  // namespace lb
