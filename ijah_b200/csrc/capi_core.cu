// C ABI, part 1: errors, dtypes, device query, buffers, packs (the reference's core/capi.mm, core/pack.mm and
// core/tensor.h surface on CUDA). Declarations and the reference lines they replace: include/ijah_engine.h.
#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <climits>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "../../include/ijah_b200.h"
#include "capi_internal.hpp"
#include "json.hpp"

namespace ijah {

std::string &last_error_ref() {
  static thread_local std::string e;
  return e;
}

// ------------------------------------------------------------------ per-device scratch + status word
// The word the kernels report bounded-wait failures into is part of the library image (zero when the library is loaded on
// a device), so neither reporting nor reading it ever allocates; every entry point, ne_exl3_linear_static included, hands
// this one word to its kernels and ne_device_wait_status() reads it.
static __device__ int g_wait_status;

struct DeviceState {
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  int *status = nullptr;
  int sms = 0;
};
static DeviceState &dev_state() {
  static std::mutex mu;
  static std::map<int, DeviceState> st;
  int d = 0;
  IJ_CUDA(cudaGetDevice(&d));
  std::lock_guard<std::mutex> lk(mu);
  return st[d];
}
void *device_scratch(size_t bytes) {
  DeviceState &s = dev_state();
  if (bytes > s.scratch_bytes) {
    if (s.scratch) {
      IJ_CUDA(cudaDeviceSynchronize());
      IJ_CUDA(cudaFree(s.scratch));
      s.scratch = nullptr;
    }
    const size_t want = std::max(bytes, (size_t)(8u << 20));
    IJ_CUDA(cudaMalloc(&s.scratch, want));
    s.scratch_bytes = want;
  }
  return s.scratch;
}
int *device_status_word() {
  DeviceState &s = dev_state();
  if (!s.status) {  // in host code the symbol is only a handle: its device address is looked up once per device
    void *p = nullptr;
    IJ_CUDA(cudaGetSymbolAddress(&p, g_wait_status));
    s.status = static_cast<int *>(p);
  }
  return s.status;
}
void check_status_word() {
  int v = 0;
  IJ_CUDA(cudaMemcpy(&v, device_status_word(), sizeof v, cudaMemcpyDeviceToHost));
  if (v != 0) {
    IJ_CUDA(cudaMemset(device_status_word(), 0, sizeof(int)));
    fail("a device-side bounded wait gave up (code %d: 1 = ring slot never freed, 2 = tiles never arrived)", v);
  }
}
void make_trellis_map(CUtensorMap *out, const void *base, int E, int IT, int OT, int K, int ks) {
  typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn encode = nullptr;  // the driver's cuTensorMapEncodeTiled, looked up through the runtime (no link against libcuda)
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    IJ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    IJ_CHECK(fn != nullptr && q == cudaDriverEntryPointSuccess, "the driver does not provide cuTensorMapEncodeTiled");
    encode = reinterpret_cast<encode_fn>(fn);
  }
  IJ_CHECK(((uintptr_t)base & 15) == 0, "trellis must be 16-byte aligned on the device");
  IJ_CHECK(E >= 1 && IT >= 1 && OT >= 1 && K >= 4 && K <= 8 && ks >= 1 && ks <= 256, "bad trellis dims for a tensor map");
  const cuuint64_t dims[3] = {(cuuint64_t)OT * 4 * K, (cuuint64_t)IT, (cuuint64_t)E};
  const cuuint64_t strides[2] = {(cuuint64_t)OT * 32 * K, (cuuint64_t)IT * OT * 32 * K};
  const cuuint32_t box[3] = {(cuuint32_t)(8 * 4 * K), (cuuint32_t)ks, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult rc = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  IJ_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed (%d) for a trellis of %d x %d x %d tiles, K%d", (int)rc, E, IT, OT, K);
}

int sm_count() {
  {
    int d0 = 0;
    if (cudaGetDevice(&d0) != cudaSuccess) {  // planning without a device (B200)
      cudaGetLastError();
      return 148;
    }
  }
  DeviceState &s = dev_state();
  if (!s.sms) {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || s.sms <= 0) {
      cudaGetLastError();
      s.sms = 148;  // planning without a device (B200)
    }
  }
  return s.sms;
}

// ------------------------------------------------------------------ buffers
void *Buf::device() {
  if (!dev && pack_host) {  // pack tensor: device copy on first use
    IJ_CUDA(cudaMalloc(&dev, std::max<uint64_t>(size, 16)));
    IJ_CUDA(cudaMemcpy(dev, pack_host, size, cudaMemcpyHostToDevice));
  }
  return dev;
}
Buf::~Buf() {
  if (dev) cudaFree(dev);
}

// ------------------------------------------------------------------ packs
static const struct { const char *name; int code; int size; } kDtypes[] = {
    {"F32", NE_F32, 4}, {"F16", NE_F16, 2}, {"BF16", NE_BF16, 2}, {"U8", NE_U8, 1},   {"U16", NE_U16, 2},
    {"U32", NE_U32, 4}, {"I32", NE_I32, 4}, {"I64", NE_I64, 8},   {"I8", NE_I8, 1},   {"I16", NE_I16, 2},
    {"U64", NE_U64, 8}, {"F64", NE_F64, 8}, {"BOOL", NE_BOOL, 1}};

static int dtype_code(const std::string &s) {
  for (auto &d : kDtypes)
    if (s == d.name) return d.code;
  fail("unknown safetensors dtype '%s'", s.c_str());
}

Shard::~Shard() {
  if (map && map != MAP_FAILED) munmap(map, bytes);
}

static std::string read_file(const std::string &path) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) return std::string();
  std::string s;
  char buf[65536];
  size_t n;
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) s.append(buf, n);
  fclose(f);
  return s;
}

static std::shared_ptr<Shard> open_shard(const std::string &path) {
  auto sh = std::make_shared<Shard>();
  char real[PATH_MAX];
  IJ_CHECK(realpath(path.c_str(), real) != nullptr, "cannot resolve %s", path.c_str());
  sh->path = real;
  const int fd = open(real, O_RDONLY);
  IJ_CHECK(fd >= 0, "cannot open %s", real);
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); fail("cannot stat %s", real); }
  sh->bytes = (size_t)st.st_size;
  if (sh->bytes < 8) { close(fd); fail("%s: too short for a safetensors file (%zu bytes)", real, sh->bytes); }
  sh->map = mmap(nullptr, sh->bytes, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  IJ_CHECK(sh->map != MAP_FAILED, "mmap %s failed", real);
  uint64_t hlen;
  memcpy(&hlen, sh->map, 8);
  IJ_CHECK(hlen <= sh->bytes - 8, "%s: header length %llu exceeds the file", real, (unsigned long long)hlen);
  sh->data_start = 8 + hlen;
  sh->header = JsonParser((const char *)sh->map + 8, hlen).parse();
  IJ_CHECK(sh->header.kind == Json::Obj, "%s: header is not an object", real);
  return sh;
}

std::shared_ptr<Pack> Pack::open(const std::string &dir) {
  auto p = std::make_shared<Pack>();
  p->dir = dir;
  p->config = read_file(dir + "/config.json");
  if (p->config.empty()) p->config = "{}";
  std::vector<std::string> files;
  const std::string idx = read_file(dir + "/model.safetensors.index.json");
  if (!idx.empty()) {
    const Json j = JsonParser(idx.data(), idx.size()).parse();
    const Json *wm = j.get("weight_map");
    IJ_CHECK(wm && wm->kind == Json::Obj, "%s: index has no weight_map", dir.c_str());
    for (auto &kv : wm->obj)
      if (std::find(files.begin(), files.end(), kv.second.str) == files.end()) files.push_back(kv.second.str);
  } else {
    DIR *d = opendir(dir.c_str());
    IJ_CHECK(d != nullptr, "cannot open pack directory %s", dir.c_str());
    while (dirent *e = readdir(d)) {
      const std::string n = e->d_name;
      if (n.size() > 12 && n.substr(n.size() - 12) == ".safetensors") files.push_back(n);
    }
    closedir(d);
    std::sort(files.begin(), files.end());
  }
  IJ_CHECK(!files.empty(), "%s: no safetensors shards", dir.c_str());
  for (auto &f : files) {
    auto sh = open_shard(dir + "/" + f);
    for (auto &kv : sh->header.obj) {
      if (kv.first == "__metadata__") continue;
      const Json &t = kv.second;
      const Json *dt = t.get("dtype"), *shp = t.get("shape"), *off = t.get("data_offsets");
      IJ_CHECK(dt && shp && off && off->arr.size() == 2, "%s: bad entry for %s", sh->path.c_str(), kv.first.c_str());
      TensorInfo ti;
      ti.name = kv.first;
      ti.dtype = dtype_code(dt->str);
      ti.ndim = (int)shp->arr.size();
      IJ_CHECK(ti.ndim <= NE_MAX_DIMS, "%s: %d dims", kv.first.c_str(), ti.ndim);
      uint64_t numel = 1;
      for (int i = 0; i < ti.ndim; i++) { ti.shape[i] = shp->arr[i].as_int(); numel *= (uint64_t)ti.shape[i]; }
      const uint64_t a = (uint64_t)off->arr[0].as_int(), b = (uint64_t)off->arr[1].as_int();
      ti.nbytes = b - a;
      IJ_CHECK(b >= a && ti.nbytes == numel * (uint64_t)ne_dtype_size(ti.dtype), "%s: size does not match shape", kv.first.c_str());
      ti.file_offset = sh->data_start + a;
      IJ_CHECK(ti.file_offset + ti.nbytes <= sh->bytes, "%s: data runs past the end of %s", kv.first.c_str(), sh->path.c_str());
      ti.shard = sh;
      ti.host = (const char *)sh->map + ti.file_offset;
      p->tensors[ti.name] = std::move(ti);
    }
    p->shards.push_back(sh);
  }
  for (auto &kv : p->tensors) p->names.push_back(kv.first);  // std::map iterates sorted by name
  return p;
}

const TensorInfo *Pack::info(const std::string &name) const {
  auto it = tensors.find(name);
  return it == tensors.end() ? nullptr : &it->second;
}

Buf *Pack::buf_of(const TensorInfo &ti) {
  std::lock_guard<std::mutex> lk(mu);
  auto it = bufs.find(ti.name);
  if (it != bufs.end()) return it->second.get();
  auto b = std::make_unique<Buf>();
  b->size = ti.nbytes;
  b->pack_host = ti.host;
  b->pack_owned = true;
  Buf *raw = b.get();
  bufs[ti.name] = std::move(b);
  return raw;
}

const void *Pack::device(const std::string &name, const TensorInfo **out) {
  const TensorInfo *ti = info(name);
  IJ_CHECK(ti != nullptr, "pack has no tensor %s", name.c_str());
  if (out) *out = ti;
  return buf_of(*ti)->device();
}

struct PackHandle {
  std::shared_ptr<Pack> pack;
};
std::shared_ptr<Pack> pack_from_c(ne_pack *p) { return p ? reinterpret_cast<PackHandle *>(p)->pack : nullptr; }

}  // namespace ijah

using namespace ijah;

extern "C" {

NE_API int ne_abi_version(void) { return NE_ABI_VERSION; }
NE_API const char *ne_last_error(void) { return last_error_ref().c_str(); }
NE_API const char *ne_dtype_name(int dtype) {
  for (auto &d : kDtypes)
    if (d.code == dtype) return d.name;
  return "?";
}
NE_API int ne_dtype_size(int dtype) {
  for (auto &d : kDtypes)
    if (d.code == dtype) return d.size;
  return 0;
}

NE_API int ne_device_query(ne_device_info *out) {
  return c_call([&] {
    IJ_CHECK(out != nullptr, "null ne_device_info");
    memset(out, 0, sizeof *out);
    int d = 0;
    IJ_CUDA(cudaGetDevice(&d));
    cudaDeviceProp pr;
    IJ_CUDA(cudaGetDeviceProperties(&pr, d));
    memcpy(out->name, pr.name, std::min(sizeof out->name - 1, strlen(pr.name)));  // the struct was zeroed: stays terminated
    out->has_nax = pr.major >= 7 ? 1 : 0;
    out->has_metal4 = 0;
    out->max_buffer_length = pr.totalGlobalMem;
    out->recommended_working_set = pr.totalGlobalMem;
    out->max_threadgroup_memory = pr.sharedMemPerBlockOptin;
    snprintf(out->backend, sizeof out->backend, "cuda");
  });
}

NE_API ne_buf *ne_alloc(uint64_t nbytes) {
  Buf *b = nullptr;
  const int rc = c_call([&] {
    auto u = std::make_unique<Buf>();
    u->size = std::max<uint64_t>(nbytes, 16);
    IJ_CUDA(cudaMallocManaged(&u->dev, u->size));
    u->managed = true;
    IJ_CUDA(cudaMemset(u->dev, 0, u->size));
    IJ_CUDA(cudaDeviceSynchronize());
    b = u.release();
  });
  return rc == 0 ? reinterpret_cast<ne_buf *>(b) : nullptr;
}
NE_API void ne_free(ne_buf *b) {
  Buf *x = reinterpret_cast<Buf *>(b);
  if (x && !x->pack_owned) delete x;
}
NE_API uint64_t ne_buf_size(const ne_buf *b) { return b ? reinterpret_cast<const Buf *>(b)->size : 0; }
NE_API void *ne_buf_contents(const ne_buf *b) {
  const Buf *x = reinterpret_cast<const Buf *>(b);
  if (!x) return nullptr;
  if (x->pack_host) return const_cast<void *>(x->pack_host);
  return x->managed ? x->dev : nullptr;
}
NE_API uint64_t ne_buf_gpu_address(const ne_buf *b) {
  uint64_t a = 0;
  c_call([&] {
    IJ_CHECK(b != nullptr, "null buffer");
    a = (uint64_t)(uintptr_t) const_cast<Buf *>(reinterpret_cast<const Buf *>(b))->device();
  });
  return a;
}
NE_API int ne_upload(ne_buf *b, uint64_t offset, const void *src, uint64_t nbytes) {
  return c_call([&] {
    Buf *x = reinterpret_cast<Buf *>(b);
    IJ_CHECK(x && src, "null argument");
    IJ_CHECK(!x->pack_owned, "ne_upload into a pack tensor is refused (read-only mapping)");
    IJ_CHECK(offset + nbytes <= x->size, "upload of %llu bytes at %llu exceeds the buffer (%llu)", (unsigned long long)nbytes,
             (unsigned long long)offset, (unsigned long long)x->size);
    IJ_CUDA(cudaMemcpy((char *)x->device() + offset, src, nbytes, cudaMemcpyHostToDevice));
  });
}
NE_API int ne_download(const ne_buf *b, uint64_t offset, void *dst, uint64_t nbytes) {
  return c_call([&] {
    Buf *x = const_cast<Buf *>(reinterpret_cast<const Buf *>(b));
    IJ_CHECK(x && dst, "null argument");
    IJ_CHECK(offset + nbytes <= x->size, "download of %llu bytes at %llu exceeds the buffer (%llu)", (unsigned long long)nbytes,
             (unsigned long long)offset, (unsigned long long)x->size);
    if (x->pack_host && !x->dev) { memcpy(dst, (const char *)x->pack_host + offset, nbytes); return; }
    IJ_CUDA(cudaMemcpy(dst, (const char *)x->device() + offset, nbytes, cudaMemcpyDeviceToHost));
  });
}

NE_API ne_pack *ne_pack_open(const char *dir) {
  PackHandle *h = nullptr;
  const int rc = c_call([&] {
    IJ_CHECK(dir != nullptr, "null directory");
    auto p = Pack::open(dir);
    h = new PackHandle{p};
  });
  return rc == 0 ? reinterpret_cast<ne_pack *>(h) : nullptr;
}
NE_API void ne_pack_close(ne_pack *p) { delete reinterpret_cast<PackHandle *>(p); }
NE_API const char *ne_pack_config_json(const ne_pack *p) {
  return p ? reinterpret_cast<const PackHandle *>(p)->pack->config.c_str() : "{}";
}
NE_API int64_t ne_pack_num_tensors(const ne_pack *p) {
  return p ? (int64_t) reinterpret_cast<const PackHandle *>(p)->pack->names.size() : 0;
}
NE_API const char *ne_pack_tensor_name(const ne_pack *p, int64_t i) {
  if (!p) return nullptr;
  auto &n = reinterpret_cast<const PackHandle *>(p)->pack->names;
  return i >= 0 && i < (int64_t)n.size() ? n[(size_t)i].c_str() : nullptr;
}
NE_API int ne_tensor_info(const ne_pack *p, const char *name, ne_tensor_desc *out) {
  return c_call([&] {
    IJ_CHECK(p && name && out, "null argument");
    Pack &pk = *reinterpret_cast<const PackHandle *>(p)->pack;
    const TensorInfo *ti = pk.info(name);
    IJ_CHECK(ti != nullptr, "no tensor named %s", name);
    memset(out, 0, sizeof *out);
    out->dtype = ti->dtype;
    out->ndim = ti->ndim;
    for (int i = 0; i < ti->ndim; i++) out->shape[i] = ti->shape[i];
    out->nbytes = ti->nbytes;
    out->file = ti->shard->path.c_str();
    out->file_offset = ti->file_offset;
    out->host = ti->host;
    out->buf = ti->nbytes ? reinterpret_cast<ne_buf *>(pk.buf_of(*ti)) : nullptr;
    out->buf_offset = 0;
  });
}
NE_API ne_buf *ne_pack_view_rows(const ne_pack *p, const char *name, int64_t row0, int64_t nrows, uint64_t *offset) {
  Buf *b = nullptr;
  const int rc = c_call([&] {
    IJ_CHECK(p && name, "null argument");
    Pack &pk = *reinterpret_cast<const PackHandle *>(p)->pack;
    const TensorInfo *ti = pk.info(name);
    IJ_CHECK(ti != nullptr, "no tensor named %s", name);
    IJ_CHECK(ti->ndim >= 1 && row0 >= 0 && nrows >= 0 && row0 + nrows <= ti->shape[0], "%s: rows [%lld, %lld) outside [0, %lld)",
             name, (long long)row0, (long long)(row0 + nrows), (long long)(ti->ndim ? ti->shape[0] : 0));
    const uint64_t rowb = ti->shape[0] ? ti->nbytes / (uint64_t)ti->shape[0] : 0;
    auto u = std::make_unique<Buf>();
    u->size = std::max<uint64_t>(rowb * (uint64_t)nrows, 16);
    IJ_CUDA(cudaMalloc(&u->dev, u->size));
    IJ_CUDA(cudaMemcpy(u->dev, (const char *)ti->host + rowb * (uint64_t)row0, rowb * (uint64_t)nrows, cudaMemcpyHostToDevice));
    if (offset) *offset = 0;
    b = u.release();
  });
  return rc == 0 ? reinterpret_cast<ne_buf *>(b) : nullptr;
}

NE_API int ne_copy_to_host(void *dst_host, const void *src_dev, uint64_t nbytes) {
  return c_call([&] {
    IJ_CHECK(dst_host && src_dev, "null argument");
    IJ_CUDA(cudaDeviceSynchronize());
    IJ_CUDA(cudaMemcpy(dst_host, src_dev, nbytes, cudaMemcpyDeviceToHost));
  });
}

NE_API int ne_device_wait_status(void) {
  int v = -1;
  c_call([&] {
    IJ_CUDA(cudaDeviceSynchronize());
    IJ_CUDA(cudaMemcpy(&v, device_status_word(), sizeof v, cudaMemcpyDeviceToHost));
  });
  return v;
}

}  // extern "C"
