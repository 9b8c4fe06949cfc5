// Ranks of one job, one process per GPU, for the parts of the façade that
// shard work across GPUs (the transformer layer). The reference is
// single-device (include/core/DeviceVector.h:88); nothing of this has a
// counterpart there.
//
// RankGroup is the interface the layer sees (a single rank needs no library);
// NcclRankGroup implements it over NCCL: the unique id travels from rank 0 to
// the others through a file both can see (the ranks of one box share /tmp),
// every collective is enqueued on the stream the caller names, so it is
// ordered with the engine's own kernels on that stream.
#pragma once
#include <chrono>
#include <cstdio>
#include <fstream>
#include <string>
#include <thread>

#include "cheddar/Cheddar.h"

namespace cheddar {

// Contiguous blocks of n items over `world` ranks, the first n % world ranks
// holding one more: [first, last) of `rank`, and the rank that holds item i.
inline std::pair<int, int> BlockOfRank(int n, int world, int rank) {
  const int base = n / world, rem = n % world;
  const int lo = rank * base + (rank < rem ? rank : rem);
  return {lo, lo + base + (rank < rem ? 1 : 0)};
}
inline int RankOfItem(int n, int world, int i) {
  for (int r = 0; r < world; r++)
    if (i < BlockOfRank(n, world, r).second) return r;
  return world - 1;
}

class RankGroup {
 public:
  virtual ~RankGroup() = default;
  int rank() const { return rank_; }
  int world() const { return world_; }
  // In-place broadcast of `bytes` device bytes at `buf` from `root`, enqueued on `stream`.
  virtual void Broadcast(void *buf, size_t bytes, int root, void *stream) {
    (void)buf, (void)bytes, (void)root, (void)stream;
  }
  // Calls between Start and End are submitted to the network together.
  virtual void Start() {}
  virtual void End() {}

 protected:
  int rank_ = 0, world_ = 1;
};

}  // namespace cheddar

#ifdef CHEDDAR_WITH_NCCL
#include <cuda_runtime_api.h>
#include <nccl.h>

namespace cheddar {

class NcclRankGroup : public RankGroup {
 public:
  // rendezvous: a path every rank can read and write; rank 0 leaves the
  // communicator's id there (and removes the file when it is destroyed)
  NcclRankGroup(int rank, int world, const std::string &rendezvous) : path_(rendezvous) {
    rank_ = rank;
    world_ = world;
    ncclUniqueId id;
    if (rank == 0) {
      Check(ncclGetUniqueId(&id), "ncclGetUniqueId");
      const std::string tmp = path_ + ".tmp";
      {
        std::ofstream f(tmp, std::ios::binary);
        f.write(reinterpret_cast<const char *>(&id), sizeof(id));
      }
      AssertTrue(std::rename(tmp.c_str(), path_.c_str()) == 0, "RankGroup: cannot publish the communicator id");
    } else {
      bool got = false;
      for (int tries = 0; tries < 1200 && !got; tries++) {  // two minutes
        std::ifstream f(path_, std::ios::binary);
        if (f && f.read(reinterpret_cast<char *>(&id), sizeof(id)) && f.gcount() == (std::streamsize)sizeof(id)) {
          got = true;
        } else {
          std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
      }
      AssertTrue(got, "RankGroup: no communicator id at " + path_);
    }
    Check(ncclCommInitRank(&comm_, world, id, rank), "ncclCommInitRank");
  }
  ~NcclRankGroup() override {
    if (comm_) ncclCommDestroy(comm_);
    if (rank_ == 0) std::remove(path_.c_str());
  }
  void Broadcast(void *buf, size_t bytes, int root, void *stream) override {
    Check(ncclBroadcast(buf, buf, bytes, ncclUint8, root, comm_, (cudaStream_t)stream), "ncclBroadcast");
  }
  void Start() override { Check(ncclGroupStart(), "ncclGroupStart"); }
  void End() override { Check(ncclGroupEnd(), "ncclGroupEnd"); }

 private:
  static void Check(ncclResult_t r, const char *what) {
    if (r != ncclSuccess) Fail(std::string(what) + ": " + ncclGetErrorString(r));
  }
  std::string path_;
  ncclComm_t comm_ = nullptr;
};

}  // namespace cheddar
#endif  // CHEDDAR_WITH_NCCL
