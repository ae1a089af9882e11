// Peer-memory collectives of the tensor-parallel decode step: parameter blocks and launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

constexpr int kPeerMaxWorld = 8;    // ranks of one NVLink domain served by these kernels
constexpr int kPeerMaxCtas = 128;   // CTAs of one collective launch (each has its own flags)
constexpr size_t kPeerFlagBytes = 2 * kPeerMaxCtas * kPeerMaxWorld * sizeof(uint32_t);
constexpr int kPeerStatusTimeout = 1;

struct PeerPointers {
  uint8_t* data[kPeerMaxWorld];     // data buffer of every rank (own one included), same size on all ranks
  uint32_t* flags[kPeerMaxWorld];   // flag array of every rank: [2 phases][kPeerMaxCtas][kPeerMaxWorld]
};

struct PeerState {                  // local device memory of this rank
  uint32_t* epoch;                  // number of collective launches completed
  unsigned int* ticket;             // CTAs of the current launch that have finished
  int32_t* status;                  // sticky status word
  unsigned int max_polls;           // bound of every flag wait (each poll sleeps >= 100 ns)
};

// In-place sum of n_elems bf16 values at byte offset `offset_bytes` of every rank's data buffer.
// n_elems must be a multiple of 8 * world.
cudaError_t launch_peer_allreduce_bf16(const PeerPointers& pp, const PeerState& st, int rank, int world,
                                       long long offset_bytes, long long n_elems, int ctas, cudaStream_t stream);

// delta = sum over ranks of the [rows, cols] bf16 region at part_off; x (region at x_off) += delta;
// h (region at h_off) = rmsnorm(x) * w, in every rank's buffer.  rows % world == 0, cols % 8 == 0, cols <= 16384.
cudaError_t launch_peer_allreduce_add_rmsnorm(const PeerPointers& pp, const PeerState& st, int rank, int world,
                                              long long part_off, long long x_off, long long h_off, int rows, int cols,
                                              const void* w, float eps, cudaStream_t stream);

// Rank r's `chunk_bytes` at `src` (local memory) end up at offset_bytes + r * chunk_bytes of every
// rank's data buffer.  chunk_bytes must be a multiple of 4.
cudaError_t launch_peer_allgather(const PeerPointers& pp, const PeerState& st, int rank, int world, const void* src,
                                  long long offset_bytes, long long chunk_bytes, cudaStream_t stream);

}  // namespace fa
