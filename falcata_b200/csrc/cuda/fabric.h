// Symmetric heap over NVLink for the in-kernel collectives of multi-GPU training.
//
// One process drives one GPU. Every rank allocates a heap of the same size, exports it as a CUDA
// IPC handle, and maps every peer's heap (NVSwitch gives each GPU full-bandwidth loads, stores and
// reductions to every peer). Regions are carved with a bump allocator in the same order on every
// rank, so an offset names the same object on all ranks. Kernels then add histogram bins straight
// into the owner's pool (red.add over NVLink), publish small records with plain stores and order
// them with release/acquire flags. torch.distributed is used only to exchange the 64-byte handles.
//
// Every wait on a peer's flag is bounded: when the spin budget runs out the kernel records
// kStatusWaitTimeout in the status word and carries on, so a missing rank can never hang a GPU.
//
// Parity: replaces include/Falcata/cuda/cuda_nccl_topology.hpp (communicator bootstrap) and the
// ncclAllReduce call sites listed for src/treelearner/cuda/cuda_single_gpu_tree_learner.cpp:L4091-4249,
// cuda_leaf_splits.cu:L356-410, cuda_gradient_discretizer.cu:L359-370, cuda_data_partition.cu:L1066-1077.
#pragma once
#include "device_common.cuh"

namespace fb {

constexpr int kMaxRanks = 8;

struct FabricView {
  int rank, world;
  char* base[kMaxRanks];            // mapped heap base of every rank (own heap at [rank])
  unsigned long long max_spins;
  unsigned int* status;             // device status word of this rank (DeviceStatus, 0 = ok)
};

// Completion signal of a multi-block producer kernel: the last block to finish raises this rank's
// flag on every peer.
struct FabricSignal {
  int world;
  unsigned int* done_counter;       // local
  unsigned int* peer_flag[kMaxRanks];   // address of flag[this rank] inside every rank's heap
  unsigned int epoch;
};

struct FabricWait {
  int world;
  const unsigned int* flags;        // local flag array, one entry per source rank
  unsigned int epoch;
  unsigned long long max_spins;
  unsigned int* status;
};

enum FabricOp : int { kFabricMaxF32 = 0, kFabricSumI64 = 1, kFabricSumF64 = 2 };

class Fabric {
 public:
  static Fabric& Get();
  bool active() const { return world_ > 1 && connected_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  // Allocate this rank's heap; returns the IPC handle to hand to the peers.
  void Create(int rank, int world, size_t bytes, char out_handle[64]);
  void Connect(const char* handles /* world x 64 bytes, by rank */);
  void Destroy();
  // Carving. Reset() starts a new layout (one engine at a time uses the heap).
  void Reset() { cursor_ = flag_bytes_; flag_cursor_ = fixed_flag_cursor_; guards_.resize(fixed_guards_); }
  size_t Alloc(size_t bytes, size_t align = 256);
  // FALCATA_DEBUG=canary: every region carved by Alloc is followed by kGuardBytes of a fixed pattern in this rank's heap;
  // CheckCanaries reads them back and returns the index (in allocation order) of the first region whose guard was
  // overwritten - by this rank or by a peer's store - or -1.
  static constexpr size_t kGuardBytes = 256;
  int CheckCanaries(cudaStream_t s) const;
  template <typename T> T* Ptr(int r, size_t off) const { return reinterpret_cast<T*>(base_[r] + off); }
  template <typename T> T* Local(size_t off) const { return Ptr<T>(rank_, off); }
  FabricView View() const;
  // Flag slots live at the start of the heap and are never reused: epochs only grow, so a stale
  // flag can never satisfy a later wait. Each call returns a fresh (flag array offset, counter).
  size_t NewFlagSlot();
  unsigned int NextEpoch() { return ++epoch_; }
  unsigned int* done_counter(int which) const { return counters_ + which; }
  unsigned int* status_word() const { return status_; }
  // Reads and clears the status word (host side, synchronises the stream).
  int CheckStatus(cudaStream_t s);
  void set_max_spins(unsigned long long v) { max_spins_ = v; }
  // Small all-reduce through the heap: every rank stores its vector into every peer, then combines.
  void AllReduce(FabricOp op, const void* src, void* dst, int count, cudaStream_t s);

 private:
  int rank_ = 0, world_ = 1;
  bool connected_ = false;
  char* base_[kMaxRanks] = {nullptr};
  size_t bytes_ = 0, cursor_ = 0, flag_bytes_ = 0, flag_cursor_ = 0, fixed_flag_cursor_ = 0;
  unsigned int epoch_ = 0;
  unsigned int* counters_ = nullptr;   // local device memory
  unsigned int* status_ = nullptr;
  unsigned long long max_spins_ = 20000000ull;
  size_t ar_data_off_ = 0, ar_flag_off_ = 0;
  std::vector<size_t> guards_;   // offsets of the guard blocks (debug mode)
  size_t fixed_guards_ = 0;      // guards of the regions that Reset() keeps
};

// Call with all threads of the block; the block's global writes are ordered before the flag.
// `wrote_peers`: this block stored into other ranks' memory. Such a block publishes its own stores at SYSTEM
// scope before it counts itself in, so the flag can never overtake data that is still on its way through
// NVLink; blocks that only wrote local memory take the cheaper device-scope fence. The last block, which has
// observed all the others through the counter, issues one more system-scope fence and raises the flags.
__device__ inline void FabricSignalDone(const FabricSignal& sig, unsigned int total_blocks, bool wrote_peers = false) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (wrote_peers) __threadfence_system(); else __threadfence();
    const unsigned int prev = atomicAdd(sig.done_counter, 1u);
    if (prev + 1 == total_blocks) {
      *sig.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < sig.world; ++r) StoreFlagAfterFence(sig.peer_flag[r], sig.epoch);
    }
  }
}

__device__ inline void FabricWaitAll(const FabricWait& w) {
  // call with all threads of the block
  if (threadIdx.x < w.world) {
    if (!WaitFlagGE(w.flags + threadIdx.x, w.epoch, w.max_spins)) atomicExch(w.status, static_cast<unsigned int>(kStatusWaitTimeout));
  }
  __syncthreads();
}

}  // namespace fb
