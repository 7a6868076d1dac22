// Types behind the opaque C handles (ne_buf, ne_pack), shared by the C ABI sources.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "common.hpp"
#include "json.hpp"

struct ne_pack;

namespace ijah {

// ne_buf: a managed allocation (ne_alloc), a device copy of pack rows (ne_pack_view_rows), or a pack tensor whose
// device copy is made on first use.
struct Buf {
  void *dev = nullptr;
  uint64_t size = 0;
  bool managed = false;
  bool pack_owned = false;
  const void *pack_host = nullptr;  // read-only file mapping of a pack tensor
  void *device();
  ~Buf();
};

struct Shard {
  std::string path;
  void *map = nullptr;
  size_t bytes = 0;
  uint64_t data_start = 0;
  Json header;
  ~Shard();
};

struct TensorInfo {
  std::string name;
  int dtype = 0, ndim = 0;
  int64_t shape[8] = {0};
  uint64_t nbytes = 0, file_offset = 0;
  const void *host = nullptr;
  std::shared_ptr<Shard> shard;
};

struct Pack {
  std::string dir, config;
  std::vector<std::shared_ptr<Shard>> shards;
  std::map<std::string, TensorInfo> tensors;
  std::vector<std::string> names;
  std::map<std::string, std::unique_ptr<Buf>> bufs;
  std::mutex mu;
  static std::shared_ptr<Pack> open(const std::string &dir);
  const TensorInfo *info(const std::string &name) const;
  Buf *buf_of(const TensorInfo &ti);
  const void *device(const std::string &name, const TensorInfo **out = nullptr);  // resident device copy
};

std::shared_ptr<Pack> pack_from_c(ne_pack *p);
struct Q8Weight;
// 8-bit affine Linear `pre`.weight / .scales / .biases of a pack, resident on the device (capi_layer.cu)
Q8Weight pack_q8(Pack &p, const std::string &pre);

}  // namespace ijah
