// Host-side C++ mirror of the reference's operator API (namespace cheddar,
// word = uint32_t) on top of the C ABI of libcheddar_b200.so.
//
// Class and method names, argument meaning and error behaviour follow the
// reference headers (include/core/Parameter.h, NPInfo.h, Container.h,
// Context.h, Encode.h, include/UserInterface.h): a size / level / scale
// violation prints a message and exits (reference include/common/Assert.h).
// Everything that touches the GPU is a call into the C ABI; this header holds
// only metadata bookkeeping and the client-side host code (sampling, CKKS
// encoding), which the reference also runs on the CPU.
#pragma once
#include <algorithm>
#include <cmath>
#include <complex>
#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <cstring>
#include <iostream>
#include <map>
#include <memory>
#include <numeric>
#include <random>
#include <sstream>
#include <string>
#include <utility>
#include <set>
#include <vector>

#include "cheddar_b200.h"

namespace cheddar {

using Complex = std::complex<double>;

// ---------------------------------------------------------------- asserts
[[noreturn]] inline void Fail(const std::string &msg) {
  std::cerr << "ERROR: " << msg << std::endl;
  std::exit(EXIT_FAILURE);
}
inline void AssertTrue(bool c, const std::string &msg) {
  if (!c) Fail(msg);
}
inline void AssertFalse(bool c, const std::string &msg) {
  if (c) Fail(msg);
}
inline void Warn(const std::string &msg) { std::clog << "WARN: " << msg << std::endl; }
inline void CheckAbi(int rc) {
  if (rc < 0) Fail(cfhe_last_error());
}

template <typename T>
T Max(T a, T b) { return a > b ? a : b; }
template <typename T>
T Min(T a, T b) { return a < b ? a : b; }
inline int DivCeil(int a, int b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------- NPInfo
struct NPInfo {
  int num_main_ = 0, num_ter_ = 0, num_aux_ = 0;
  NPInfo(int num_main = 0, int num_ter = 0, int num_aux = 0)
      : num_main_{num_main}, num_ter_{num_ter}, num_aux_{num_aux} {
    AssertTrue(num_main >= 0 && num_ter >= 0 && num_aux >= 0, "Negative prime count given");
  }
  int GetNumQ() const { return num_main_ + num_ter_; }
  int GetNumTotal() const { return num_main_ + num_ter_ + num_aux_; }
  bool operator==(const NPInfo &o) const {
    return num_main_ == o.num_main_ && num_ter_ == o.num_ter_ && num_aux_ == o.num_aux_;
  }
  bool IsSubsetOf(const NPInfo &o) const {
    return num_main_ <= o.num_main_ && num_ter_ <= o.num_ter_ && num_aux_ <= o.num_aux_;
  }
  bool IsSupersetOf(const NPInfo &o) const { return o.IsSubsetOf(*this); }
};

// ---------------------------------------------------------------- Parameter
template <typename word>
class Parameter {
 public:
  Parameter(int log_degree, double base_scale, int default_encryption_level,
            std::vector<std::pair<int, int>> level_config, const std::vector<word> &main_primes,
            const std::vector<word> &aux_primes, const std::vector<word> &ter_primes = {},
            const std::pair<int, int> &additional_base = {0, 0})
      : log_degree_{log_degree},
        degree_{1 << log_degree},
        dnum_{DivCeil(main_primes.size() + ter_primes.size(), aux_primes.size())},
        L_{static_cast<int>(main_primes.size() + ter_primes.size())},
        alpha_{static_cast<int>(aux_primes.size())},
        base_scale_{base_scale},
        default_encryption_level_{default_encryption_level},
        max_level_{static_cast<int>(level_config.size()) - 1},
        main_primes_{main_primes},
        ter_primes_{ter_primes},
        aux_primes_{aux_primes},
        level_config_{level_config},
        additional_base_{additional_base},
        dense_h_{1 << (log_degree - 1)},
        sparse_h_{32} {
    const word ntt_base = degree_ * 2;
    auto check = [&](word p) {
      AssertTrue(p < (word(1) << 31), "Max prime is too large for the word size");
      AssertTrue(p % ntt_base == 1, "Prime is not NTT-friendly");
    };
    for (word p : main_primes_) check(p);
    for (word p : aux_primes_) check(p);
    for (word p : ter_primes_) check(p);
    AssertTrue(level_config_.back().first == (int)main_primes_.size() &&
                   level_config_.back().second == (int)ter_primes_.size(),
               "The last level should contain all the main and terminal primes");
    const int max_num_slots = degree_ / 2, m = degree_ * 2;
    galois_factors_.assign(max_num_slots + 1, 1);
    for (int i = 1; i < max_num_slots; i++)
      galois_factors_[i] = (int)(((int64_t)galois_factors_[i - 1] * 5) % m);
    q_primes_.insert(q_primes_.end(), ter_primes_.rbegin(), ter_primes_.rend());
    q_primes_.insert(q_primes_.end(), main_primes_.begin(), main_primes_.end());
    short_base_np_ = NPInfo(level_config_.at(0).first - additional_base_.first,
                            level_config_.at(0).second - additional_base_.second, 0);
    short_base_np_.num_aux_ = short_base_np_.num_main_ + short_base_np_.num_ter_;
    // Rational rescaling: going from level i to i - 1 divides by the primes
    // level i holds and level i - 1 does not and multiplies by those only the
    // lower level holds. Levels up to the default encryption level keep
    // scale_i^2 / ratio_i = scale_(i-1), i.e. scale_i = sqrt(scale_(i-1) * ratio_i)
    // (reference src/core/Parameter.cu:100-194 computes the same ratios).
    auto prime_product = [](const std::vector<word> &primes, int from, int to) {
      double p = 1.0;
      for (int j = from; j < to; j++) p *= (double)primes[j];
      return p;
    };
    rescale_prime_prod_.assign(max_level_ + 1, 0.0);
    scale_.assign(default_encryption_level_ + 1, base_scale_);
    for (int i = 1; i <= max_level_; i++) {
      const NPInfo up = LevelToNP(i), lo = LevelToNP(i - 1);
      const double gained = prime_product(ter_primes_, lo.num_ter_, up.num_ter_) *
                            prime_product(main_primes_, lo.num_main_, up.num_main_);
      const double given_back = prime_product(ter_primes_, up.num_ter_, lo.num_ter_) *
                                prime_product(main_primes_, up.num_main_, lo.num_main_);
      rescale_prime_prod_[i] = gained / given_back;
      if (i <= default_encryption_level_) scale_[i] = std::sqrt(scale_[i - 1] * rescale_prime_prod_[i]);
    }
  }

  const int log_degree_, degree_, dnum_, L_, alpha_;
  const double base_scale_;
  const int default_encryption_level_, max_level_;
  const std::vector<word> main_primes_, ter_primes_, aux_primes_;
  const std::vector<std::pair<int, int>> level_config_;
  const std::pair<int, int> additional_base_;

  int GetGaloisFactor(int i) const {
    AssertTrue(i >= 0 && i <= degree_ / 2, "GetGaloisFactor: Invalid Galois factor index");
    return galois_factors_.at(i);
  }
  double GetScale(int level) const {
    if (level == -1) level = 0;
    AssertTrue(level >= 0 && level <= default_encryption_level_, "GetScale: Invalid level");
    return scale_.at(level);
  }
  double GetRescalePrimeProd(int level) const {
    AssertTrue(level > 0 && level <= max_level_, "GetRescalePrimeProd: Invalid level");
    return rescale_prime_prod_.at(level);
  }
  int GetDenseHammingWeight() const { return dense_h_; }
  int GetSparseHammingWeight() const { return sparse_h_; }
  void SetDenseHammingWeight(int h) {
    AssertTrue(h >= sparse_h_ && h <= degree_, "SetDenseHammingWeight: invalid weight");
    dense_h_ = h;
  }
  void SetSparseHammingWeight(int h) {
    AssertTrue(h > 0 && h <= dense_h_, "SetSparseHammingWeight: invalid weight");
    sparse_h_ = h;
  }
  bool IsUsingSparseSecretEncapsulation() const { return dense_h_ > sparse_h_; }
  int GetMaxNumTer() const { return ter_primes_.size(); }
  int GetMaxNumMain() const { return main_primes_.size(); }
  int GetMaxNumQ() const { return L_; }
  int GetMaxNumAux() const { return alpha_; }
  NPInfo LevelToNP(int level, int num_aux = 0) const {
    AssertTrue(num_aux >= 0 && num_aux <= alpha_, "Invalid number of aux primes");
    if (level == -1) return NPInfo(short_base_np_.num_main_, short_base_np_.num_ter_, num_aux);
    const auto &c = level_config_.at(level);
    return NPInfo(c.first, c.second, num_aux);
  }
  int NPToLevel(const NPInfo &np) const {
    for (int i = 0; i <= max_level_; i++)
      if (level_config_[i].first == np.num_main_ && level_config_[i].second == np.num_ter_) return i;
    if (np.num_main_ == short_base_np_.num_main_ && np.num_ter_ == short_base_np_.num_ter_) return -1;
    Fail("NPInfo not found");
  }
  std::vector<word> GetPrimeVector(const NPInfo &np) const {
    std::vector<word> r(q_primes_.begin() + GetMaxNumTer() - np.num_ter_,
                        q_primes_.begin() + GetMaxNumTer() + np.num_main_);
    r.insert(r.end(), aux_primes_.begin(), aux_primes_.begin() + np.num_aux_);
    return r;
  }
  // global prime indices of the limbs of `np` (this engine's limb lists)
  std::vector<int> GetLimbIndices(const NPInfo &np) const {
    std::vector<int> g;
    for (int i = GetMaxNumTer() - np.num_ter_; i < GetMaxNumTer() + np.num_main_; i++) g.push_back(i);
    for (int a = 0; a < np.num_aux_; a++) g.push_back(L_ + a);
    return g;
  }

 private:
  std::vector<int> galois_factors_;
  std::vector<word> q_primes_;
  NPInfo short_base_np_;
  std::vector<double> rescale_prime_prod_, scale_;
  int dense_h_, sparse_h_;
};

// JSON keys of the reference's test fixture (unittest/Testbed.h:103-210).
struct ParameterJson {
  int log_degree = 0, log_default_scale = 0, default_encryption_level = 0;
  std::vector<uint32_t> main_primes, terminal_primes, auxiliary_primes;
  std::vector<std::pair<int, int>> level_config;
  std::pair<int, int> additional_base{0, 0};
  int dense_hamming_weight = -1, sparse_hamming_weight = -1;
  bool boot = false;
  int num_cts_levels = 0, num_stc_levels = 0;
};

namespace detail {
inline std::vector<long long> JsonInts(const std::string &s, const std::string &key, bool required) {
  std::vector<long long> out;
  size_t p = s.find("\"" + key + "\"");
  if (p == std::string::npos) {
    AssertFalse(required, "Missing " + key + " in JSON file");
    return out;
  }
  p = s.find(':', p) + 1;
  while (p < s.size() && isspace((unsigned char)s[p])) p++;
  auto read_num = [&](size_t &i) {
    size_t j = i;
    while (j < s.size() && (isdigit((unsigned char)s[j]) || s[j] == '-')) j++;
    out.push_back(std::stoll(s.substr(i, j - i)));
    i = j;
  };
  if (s[p] != '[') {
    if (s.compare(p, 4, "true") == 0) out.push_back(1);
    else if (s.compare(p, 5, "false") == 0) out.push_back(0);
    else read_num(p);
    return out;
  }
  int depth = 0;
  for (size_t i = p; i < s.size();) {
    if (s[i] == '[') { depth++; i++; }
    else if (s[i] == ']') { depth--; i++; if (depth == 0) break; }
    else if (isdigit((unsigned char)s[i]) || s[i] == '-') read_num(i);
    else i++;
  }
  return out;
}
}  // namespace detail

inline ParameterJson LoadParameterJson(const std::string &path) {
  std::ifstream f(path);
  AssertTrue(f.is_open(), "Failed to open JSON file: " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string s = ss.str();
  ParameterJson j;
  using detail::JsonInts;
  j.log_degree = (int)JsonInts(s, "log_degree", true)[0];
  j.log_default_scale = (int)JsonInts(s, "log_default_scale", true)[0];
  j.default_encryption_level = (int)JsonInts(s, "default_encryption_level", true)[0];
  for (auto v : JsonInts(s, "main_primes", true)) j.main_primes.push_back((uint32_t)v);
  for (auto v : JsonInts(s, "terminal_primes", false)) j.terminal_primes.push_back((uint32_t)v);
  for (auto v : JsonInts(s, "auxiliary_primes", true)) j.auxiliary_primes.push_back((uint32_t)v);
  auto lc = JsonInts(s, "level_config", true);
  AssertTrue(lc.size() % 2 == 0, "level_config should be an array of pairs");
  for (size_t i = 0; i < lc.size(); i += 2) j.level_config.emplace_back((int)lc[i], (int)lc[i + 1]);
  auto ab = JsonInts(s, "additional_base", false);
  if (ab.size() == 2) j.additional_base = {(int)ab[0], (int)ab[1]};
  auto dh = JsonInts(s, "dense_hamming_weight", false);
  if (!dh.empty()) j.dense_hamming_weight = (int)dh[0];
  auto sh = JsonInts(s, "sparse_hamming_weight", false);
  if (!sh.empty()) j.sparse_hamming_weight = (int)sh[0];
  auto b = JsonInts(s, "boot", false);
  j.boot = !b.empty() && b[0];
  auto c1 = JsonInts(s, "num_cts_levels", false);
  if (!c1.empty()) j.num_cts_levels = (int)c1[0];
  auto c2 = JsonInts(s, "num_stc_levels", false);
  if (!c2.empty()) j.num_stc_levels = (int)c2[0];
  return j;
}

template <typename word>
std::unique_ptr<Parameter<word>> MakeParameter(const ParameterJson &j) {
  auto p = std::make_unique<Parameter<word>>(
      j.log_degree, (double)(UINT64_C(1) << j.log_default_scale), j.default_encryption_level,
      j.level_config, std::vector<word>(j.main_primes.begin(), j.main_primes.end()),
      std::vector<word>(j.auxiliary_primes.begin(), j.auxiliary_primes.end()),
      std::vector<word>(j.terminal_primes.begin(), j.terminal_primes.end()), j.additional_base);
  if (j.dense_hamming_weight > 0) p->SetDenseHammingWeight(j.dense_hamming_weight);
  if (j.sparse_hamming_weight > 0) p->SetSparseHammingWeight(j.sparse_hamming_weight);
  return p;
}

// ---------------------------------------------------------------- device memory
namespace detail {
// The context new containers of this thread allocate from. Per thread: a
// host thread drives one context at a time (worker threads of a parallel
// stage each set their own with ScopedCurrentHandle).
inline cfhe_context *&CurrentHandle() {
  static thread_local cfhe_context *h = nullptr;
  return h;
}
// engines that are alive: a vector outliving its engine has nothing left to free
inline std::set<cfhe_context *> &LiveHandles() {
  static std::set<cfhe_context *> s;
  return s;
}
}  // namespace detail

// Containers created inside the scope allocate from `h` (a second context
// working beside the main one on its own stream).
class ScopedCurrentHandle {
 public:
  explicit ScopedCurrentHandle(cfhe_context *h) : saved_(detail::CurrentHandle()) {
    detail::CurrentHandle() = h;
  }
  ~ScopedCurrentHandle() { detail::CurrentHandle() = saved_; }
  ScopedCurrentHandle(const ScopedCurrentHandle &) = delete;
  ScopedCurrentHandle &operator=(const ScopedCurrentHandle &) = delete;

 private:
  cfhe_context *saved_;
};

// Move-only owner of device words (the reference's DeviceVector wraps
// rmm::device_uvector, include/core/DeviceVector.h:81-92).
template <typename word>
class DeviceVector {
 public:
  explicit DeviceVector(int size = 0) { resize(size); }
  DeviceVector(DeviceVector &&o) noexcept
      : data_(o.data_), size_(o.size_), cap_(o.cap_), owner_(o.owner_) {
    o.data_ = nullptr;
    o.size_ = o.cap_ = 0;
  }
  DeviceVector &operator=(DeviceVector &&o) noexcept {
    if (this != &o) {
      release();
      data_ = o.data_;
      size_ = o.size_;
      cap_ = o.cap_;
      owner_ = o.owner_;
      o.data_ = nullptr;
      o.size_ = o.cap_ = 0;
    }
    return *this;
  }
  DeviceVector(const DeviceVector &) = delete;
  DeviceVector &operator=(const DeviceVector &) = delete;
  ~DeviceVector() { release(); }
  void resize(int size) {  // contents are not preserved
    if (size <= cap_) {
      size_ = size;
      return;
    }
    release();
    void *p = nullptr;
    owner_ = detail::CurrentHandle();
    CheckAbi(cfhe_malloc(owner_, &p, (size_t)size * sizeof(word)));
    data_ = static_cast<word *>(p);
    size_ = cap_ = size;
  }
  word *data() { return data_; }
  const word *data() const { return data_; }
  int size() const { return size_; }

 private:
  void release() {
    // back to the allocation cache it came from (reuse there is ordered on that
    // context's stream)
    if (data_ && detail::LiveHandles().count(owner_)) cfhe_free(owner_, data_);
    data_ = nullptr;
    size_ = cap_ = 0;
  }
  word *data_ = nullptr;
  int size_ = 0, cap_ = 0;
  cfhe_context *owner_ = nullptr;
};

template <typename word>
void CopyHostToDevice(DeviceVector<word> &dst, const std::vector<word> &src) {
  dst.resize(src.size());
  CheckAbi(cfhe_copy_h2d(detail::CurrentHandle(), dst.data(), src.data(), src.size() * sizeof(word)));
  CheckAbi(cfhe_synchronize(detail::CurrentHandle()));
}
template <typename word>
void CopyDeviceToHost(std::vector<word> &dst, const DeviceVector<word> &src) {
  dst.resize(src.size());
  CheckAbi(cfhe_copy_d2h(detail::CurrentHandle(), dst.data(), src.data(), dst.size() * sizeof(word)));
}

// ---------------------------------------------------------------- containers
template <typename word>
class Container {
 protected:
  static inline int degree_ = 0;
  double scale_ = 1.0;
  NPInfo num_primes_;

 public:
  explicit Container(const NPInfo &np = NPInfo{}) : num_primes_{np} {}
  Container(Container &&) = default;
  Container &operator=(Container &&) = default;
  virtual ~Container() = default;
  virtual NPInfo GetNP() const { return num_primes_; }
  virtual void ModifyNP(const NPInfo &np) = 0;
  double GetScale() const { return scale_; }
  void SetScale(double s) { scale_ = s; }
  static void SetDegree(int d) { degree_ = d; }
  static int Degree() { return degree_; }
};

template <typename word>
class Constant : public Container<word> {
 public:
  explicit Constant(const NPInfo &np = NPInfo{}) : Container<word>(np) {}
  Constant(Constant &&) = default;
  Constant &operator=(Constant &&) = default;
  std::vector<word> cx_;  // per-limb words in M-form, kept on the host (kernel parameters)
  void ModifyNP(const NPInfo &np) override {
    this->num_primes_ = np;
    cx_.resize(np.GetNumTotal());
  }
};

template <typename word>
class Plaintext : public Container<word> {
  int num_slots_ = Container<word>::degree_ / 2;

 public:
  explicit Plaintext(const NPInfo &np = NPInfo{}) : Container<word>(np) { ModifyNP(np); }
  Plaintext(Plaintext &&) = default;
  Plaintext &operator=(Plaintext &&) = default;
  DeviceVector<word> mx_;
  void ModifyNP(const NPInfo &np) override {
    this->num_primes_ = np;
    mx_.resize(np.GetNumTotal() * Container<word>::degree_);
  }
  int GetNumSlots() const { return num_slots_; }
  void SetNumSlots(int n) { num_slots_ = n; }
};

template <typename word>
class Ciphertext : public Container<word> {
  int num_slots_ = Container<word>::degree_ / 2;
  bool has_rx_ = false;

 public:
  explicit Ciphertext(const NPInfo &np = NPInfo{}, bool has_rx = false) : Container<word>(np) {
    has_rx_ = has_rx;
    ModifyNP(np);
  }
  Ciphertext(Ciphertext &&) = default;
  Ciphertext &operator=(Ciphertext &&) = default;
  DeviceVector<word> bx_, ax_, rx_;
  bool HasRx() const { return has_rx_; }
  void PrepareRx() {
    has_rx_ = true;
    rx_.resize(this->num_primes_.GetNumTotal() * Container<word>::degree_);
  }
  void RemoveRx() {
    has_rx_ = false;
    rx_.resize(0);
  }
  void ModifyNP(const NPInfo &np) override {
    this->num_primes_ = np;
    const int n = np.GetNumTotal() * Container<word>::degree_;
    bx_.resize(n);
    ax_.resize(n);
    if (has_rx_) rx_.resize(n);
  }
  int GetNumSlots() const { return num_slots_; }
  void SetNumSlots(int n) { num_slots_ = n; }
};

template <typename word>
class EvaluationKey : public Container<word> {
 public:
  explicit EvaluationKey(const NPInfo &np = NPInfo{}, int beta = 0) : Container<word>(np) {
    for (int i = 0; i < beta; i++) {
      bx_.emplace_back(np.GetNumTotal() * Container<word>::degree_);
      ax_.emplace_back(np.GetNumTotal() * Container<word>::degree_);
    }
  }
  EvaluationKey(EvaluationKey &&) = default;
  EvaluationKey &operator=(EvaluationKey &&) = default;
  std::vector<DeviceVector<word>> bx_, ax_;
  int GetBeta() const { return bx_.size(); }
  void ModifyNP(const NPInfo &) override { Fail("EvaluationKey::ModifyNP is not supported"); }
};

// ---------------------------------------------------------------- wire format
// Ciphertexts, plaintexts and evaluation keys as byte streams (the reference
// has no serialisation: its containers live and die in one process). Layout,
// little endian: "CFHE", u32 version = 1, u32 kind (1 ciphertext, 2 plaintext,
// 3 evaluation key), u32 bytes per word, u32 ring degree, i32 num_main,
// num_ter, num_aux, f64 scale, i32 num_slots, u32 polynomial count, then the
// polynomials limb-major, words exactly as they lie in device memory
// (evaluation domain, M-form): b, a[, r] for a ciphertext; b_0, a_0, b_1, a_1,
// ... for a key. A reader checks the header against its own ring.
namespace detail {
struct WireHeader {
  char magic[4];
  uint32_t version, kind, word_bytes, degree;
  int32_t num_main, num_ter, num_aux;
  double scale;
  int32_t num_slots;
  uint32_t polys;
};
template <typename word>
void WritePoly(std::ostream &os, const DeviceVector<word> &v) {
  std::vector<word> host;
  CopyDeviceToHost(host, v);
  CheckAbi(cfhe_synchronize(CurrentHandle()));
  os.write(reinterpret_cast<const char *>(host.data()), (std::streamsize)(host.size() * sizeof(word)));
}
template <typename word>
void ReadPoly(std::istream &is, DeviceVector<word> &v, size_t words) {
  std::vector<word> host(words);
  is.read(reinterpret_cast<char *>(host.data()), (std::streamsize)(words * sizeof(word)));
  AssertTrue((size_t)is.gcount() == words * sizeof(word), "wire format: truncated stream");
  CopyHostToDevice(v, host);
}
template <typename word>
void WriteHeader(std::ostream &os, uint32_t kind, const NPInfo &np, double scale, int num_slots, uint32_t polys) {
  WireHeader h{{'C', 'F', 'H', 'E'}, 1u, kind, (uint32_t)sizeof(word), (uint32_t)Container<word>::Degree(),
               np.num_main_, np.num_ter_, np.num_aux_, scale, num_slots, polys};
  os.write(reinterpret_cast<const char *>(&h), sizeof(h));
}
template <typename word>
WireHeader ReadHeader(std::istream &is, uint32_t kind) {
  WireHeader h;
  is.read(reinterpret_cast<char *>(&h), sizeof(h));
  AssertTrue((size_t)is.gcount() == sizeof(h) && !std::memcmp(h.magic, "CFHE", 4) && h.version == 1,
             "wire format: not a container stream");
  AssertTrue(h.kind == kind, "wire format: another kind of container");
  AssertTrue(h.word_bytes == sizeof(word) && (int)h.degree == Container<word>::Degree(),
             "wire format: written for another ring");
  return h;
}
}  // namespace detail

template <typename word>
void Save(std::ostream &os, const Ciphertext<word> &ct) {
  detail::WriteHeader<word>(os, 1, ct.GetNP(), ct.GetScale(), ct.GetNumSlots(), ct.HasRx() ? 3 : 2);
  detail::WritePoly(os, ct.bx_);
  detail::WritePoly(os, ct.ax_);
  if (ct.HasRx()) detail::WritePoly(os, ct.rx_);
}
template <typename word>
void Load(std::istream &is, Ciphertext<word> &ct) {
  const auto h = detail::ReadHeader<word>(is, 1);
  AssertTrue(h.polys == 2 || h.polys == 3, "wire format: bad polynomial count");
  const NPInfo np(h.num_main, h.num_ter, h.num_aux);
  const size_t words = (size_t)np.GetNumTotal() * h.degree;
  Ciphertext<word> out(np, h.polys == 3);
  detail::ReadPoly(is, out.bx_, words);
  detail::ReadPoly(is, out.ax_, words);
  if (h.polys == 3) detail::ReadPoly(is, out.rx_, words);
  out.SetScale(h.scale);
  out.SetNumSlots(h.num_slots);
  ct = std::move(out);
}
template <typename word>
void Save(std::ostream &os, const Plaintext<word> &pt) {
  detail::WriteHeader<word>(os, 2, pt.GetNP(), pt.GetScale(), pt.GetNumSlots(), 1);
  detail::WritePoly(os, pt.mx_);
}
template <typename word>
void Load(std::istream &is, Plaintext<word> &pt) {
  const auto h = detail::ReadHeader<word>(is, 2);
  const NPInfo np(h.num_main, h.num_ter, h.num_aux);
  Plaintext<word> out(np);
  detail::ReadPoly(is, out.mx_, (size_t)np.GetNumTotal() * h.degree);
  out.SetScale(h.scale);
  out.SetNumSlots(h.num_slots);
  pt = std::move(out);
}
template <typename word>
void Save(std::ostream &os, const EvaluationKey<word> &key) {
  detail::WriteHeader<word>(os, 3, key.GetNP(), key.GetScale(), 0, 2 * (uint32_t)key.GetBeta());
  for (int j = 0; j < key.GetBeta(); j++) {
    detail::WritePoly(os, key.bx_[j]);
    detail::WritePoly(os, key.ax_[j]);
  }
}
template <typename word>
void Load(std::istream &is, EvaluationKey<word> &key) {
  const auto h = detail::ReadHeader<word>(is, 3);
  AssertTrue(h.polys % 2 == 0, "wire format: bad polynomial count");
  const NPInfo np(h.num_main, h.num_ter, h.num_aux);
  EvaluationKey<word> out(np, (int)h.polys / 2);
  for (int j = 0; j < (int)h.polys / 2; j++) {
    detail::ReadPoly(is, out.bx_[j], (size_t)np.GetNumTotal() * h.degree);
    detail::ReadPoly(is, out.ax_[j], (size_t)np.GetNumTotal() * h.degree);
  }
  out.SetScale(h.scale);
  key = std::move(out);
}

// ---------------------------------------------------------------- random
// Same distributions as the reference's Random (include/Random.h:16-81); the
// generator is seedable here (the reference's is not).
class Random {
 public:
  static void Seed(uint64_t s) { gen_.seed(s); }
  static uint64_t Draw64() { return gen_(); }
  template <typename word>
  static void SampleUniformWord(word *p, int n, word lo, word hi) {
    std::uniform_int_distribution<word> d(lo, hi);
    std::generate(p, p + n, [&]() { return d(gen_); });
  }
  // Uniform residues in [0, q): both 32-bit halves of every generator output
  // are used, each mapped to the range by the multiply-and-reject method
  // (exactly uniform), several times faster than a distribution object per word.
  static void SampleUniformBelow(uint32_t *p, size_t n, uint32_t q) {
    const uint32_t reject_below = (uint32_t)(0u - q) % q;  // 2^32 mod q
    uint64_t pool = 0;
    int have = 0;
    for (size_t i = 0; i < n;) {
      if (!have) {
        pool = gen_();
        have = 2;
      }
      const uint32_t r = (uint32_t)pool;
      pool >>= 32;
      have--;
      const uint64_t m = (uint64_t)r * q;
      if ((uint32_t)m >= reject_below) p[i++] = (uint32_t)(m >> 32);
    }
  }
  static void SampleWithoutReplacement(int *p, int n, int lo, int hi) {
    AssertTrue(hi - lo + 1 >= n, "Invalid length");
    std::vector<int> v(hi - lo + 1);
    std::iota(v.begin(), v.end(), lo);
    std::shuffle(v.begin(), v.end(), gen_);
    std::copy(v.begin(), v.begin() + n, p);
  }
  static void SampleUniformComplex(Complex *p, int n, double lo, double hi) {
    std::uniform_real_distribution<double> d(lo, hi);
    std::generate(p, p + n, [&]() { return Complex(d(gen_), d(gen_)); });
  }
  static void SampleDiscreteNormal(int *p, int n, double mean, double stddev, double max_sigma = 6) {
    std::normal_distribution<double> d(0, stddev);
    std::generate(p, p + n, [&]() {
      double v = d(gen_);
      v = std::min(std::max(v, -max_sigma * stddev), max_sigma * stddev);
      return (int)std::llround(v + mean);
    });
  }

 private:
  static inline std::mt19937_64 gen_{0xC0FFEE};
};

// ---------------------------------------------------------------- big unsigned
namespace detail {
// little-endian base-2^32 unsigned integer, just enough for CRT reconstruction
struct BigU {
  std::vector<uint32_t> w;
  explicit BigU(size_t n = 0) : w(n, 0) {}
  void mul_small(uint32_t m) {
    uint64_t c = 0;
    for (auto &x : w) {
      c += (uint64_t)x * m;
      x = (uint32_t)c;
      c >>= 32;
    }
    if (c) w.push_back((uint32_t)c);
  }
  void add_mul(const BigU &o, uint32_t m) {  // this += o * m
    if (w.size() < o.w.size() + 2) w.resize(o.w.size() + 2, 0);
    uint64_t c = 0;
    size_t i = 0;
    for (; i < o.w.size(); i++) {
      c += (uint64_t)o.w[i] * m + w[i];
      w[i] = (uint32_t)c;
      c >>= 32;
    }
    for (; c && i < w.size(); i++) {
      c += w[i];
      w[i] = (uint32_t)c;
      c >>= 32;
    }
  }
  int cmp(const BigU &o) const {
    size_t n = std::max(w.size(), o.w.size());
    for (size_t i = n; i-- > 0;) {
      uint32_t a = i < w.size() ? w[i] : 0, b = i < o.w.size() ? o.w[i] : 0;
      if (a != b) return a < b ? -1 : 1;
    }
    return 0;
  }
  void sub(const BigU &o) {  // requires *this >= o
    int64_t br = 0;
    for (size_t i = 0; i < w.size(); i++) {
      int64_t d = (int64_t)w[i] - (i < o.w.size() ? o.w[i] : 0) - br;
      br = d < 0;
      w[i] = (uint32_t)(d + (br << 32));
    }
  }
  double to_double() const {
    double r = 0;
    for (size_t i = w.size(); i-- > 0;) r = r * 4294967296.0 + w[i];
    return r;
  }
  BigU half() const {
    BigU r(w.size());
    for (size_t i = 0; i < w.size(); i++)
      r.w[i] = (w[i] >> 1) | (i + 1 < w.size() ? (w[i + 1] << 31) : 0);
    return r;
  }
};
inline uint32_t MulMod(uint32_t a, uint32_t b, uint32_t q) { return (uint32_t)((uint64_t)a * b % q); }
inline uint32_t PowMod(uint32_t a, uint64_t e, uint32_t q) {
  uint32_t r = 1;
  for (a %= q; e; e >>= 1, a = MulMod(a, a, q))
    if (e & 1) r = MulMod(r, a, q);
  return r;
}
inline uint32_t InvMod(uint32_t a, uint32_t q) { return PowMod(a, (uint64_t)q - 2, q); }
inline uint32_t ToMontgomery(uint32_t a, uint32_t q) { return (uint32_t)(((uint64_t)a << 32) % q); }
inline uint32_t ModI128(__int128 v, uint32_t q) {
  __int128 r = v % (__int128)q;
  if (r < 0) r += q;
  return (uint32_t)r;
}
}  // namespace detail

template <typename word>
class Context;
template <typename word>
using ContextPtr = std::shared_ptr<Context<word>>;
template <typename word>
using ConstContextPtr = std::shared_ptr<const Context<word>>;

// ---------------------------------------------------------------- Encoder
// CKKS encoding on the host (reference src/core/Encode.cpp); only the final
// NTT / INTT runs on the GPU, as in the reference.
template <typename word>
class Encoder {
 public:
  Encoder(const Parameter<word> &param, cfhe_context *h) : param_{param}, h_{h}, M_{param.degree_ * 2} {
    twiddle_factors_.resize(M_);
    for (int i = 0; i < M_; i++) twiddle_factors_[i] = std::polar(1.0, 2.0 * M_PI * i / M_);
  }

  void Encode(Plaintext<word> &ptxt, int level, double scale, const std::vector<Complex> &message,
              int num_aux = 0) const {
    int num_slots = 1;
    while (num_slots < (int)message.size()) num_slots <<= 1;
    std::vector<Complex> data(num_slots);
    std::copy(message.begin(), message.end(), data.begin());
    SpecialIFFT(data);
    const int degree = param_.degree_, half = degree / 2, gap = half / num_slots;
    AssertTrue(num_slots <= half, "Encode: Too many slots");
    NPInfo np = param_.LevelToNP(level, num_aux);
    const int nt = np.GetNumTotal();
    // coefficients times the scale; the engine truncates them toward zero (as
    // the reference's BigInt(double) does), reduces them modulo every prime of
    // the level and transforms the limbs, all on the device
    std::vector<double> coeffs(degree, 0.0);
    for (int i = 0; i < num_slots; i++) {
      coeffs[(size_t)i * gap] = data[i].real() * scale;
      coeffs[(size_t)i * gap + half] = data[i].imag() * scale;
    }
    ptxt.ModifyNP(np);
    ptxt.SetNumSlots(num_slots);
    ptxt.SetScale(scale);
    auto g = param_.GetLimbIndices(np);
    CheckAbi(cfhe_encode_coeffs(h_, ptxt.mx_.data(), coeffs.data(), g.data(), nt));
  }

  // The centred integer coefficients are rebuilt on the device
  // (cfhe_decode_coeffs: fractions find the multiple of Q, 128-bit wrapping
  // arithmetic the value); DecodeOnHost is the big-integer form of the same
  // lift (the reference's, src/core/Encode.cpp:250-275).
  void Decode(std::vector<Complex> &message, const Plaintext<word> &ptxt) const {
    NPInfo np = ptxt.GetNP();
    AssertTrue(np.num_aux_ == 0, "Decode: Aux primes not supported");
    auto primes = param_.GetPrimeVector(np);
    const int nt = np.GetNumTotal(), degree = param_.degree_, half = degree / 2;
    const int num_slots = ptxt.GetNumSlots(), gap = half / num_slots;
    std::vector<word> icrt = InverseCrtConstants(primes, degree);
    // (Q / q_j) and Q modulo 2^128
    std::vector<uint32_t> hat((size_t)4 * nt, 0), q_low(4, 0);
    auto low_words = [](const detail::BigU &b, uint32_t *dst) {
      for (size_t w = 0; w < 4; w++) dst[w] = w < b.w.size() ? b.w[w] : 0;
    };
    detail::BigU Q(1);
    Q.w[0] = 1;
    for (int j = 0; j < nt; j++) {
      Q.mul_small(primes[j]);
      detail::BigU h(1);
      h.w[0] = 1;
      for (int k = 0; k < nt; k++)
        if (k != j) h.mul_small(primes[k]);
      low_words(h, &hat[(size_t)4 * j]);
    }
    low_words(Q, q_low.data());
    std::vector<double> coeffs(degree);
    auto g = param_.GetLimbIndices(np);
    CheckAbi(cfhe_decode_coeffs(h_, coeffs.data(), ptxt.mx_.data(), g.data(), nt, icrt.data(), hat.data(),
                                q_low.data()));
    message.resize(num_slots);
    const double scale = ptxt.GetScale();
    for (int i = 0; i < num_slots; i++)
      message[i] = Complex(coeffs[(size_t)i * gap] / scale, coeffs[(size_t)i * gap + half] / scale);
    SpecialFFT(message);
  }

  void DecodeOnHost(std::vector<Complex> &message, const Plaintext<word> &ptxt) const {
    NPInfo np = ptxt.GetNP();
    AssertTrue(np.num_aux_ == 0, "Decode: Aux primes not supported");
    auto primes = param_.GetPrimeVector(np);
    const int nt = np.GetNumTotal(), degree = param_.degree_, half = degree / 2;
    const int num_slots = ptxt.GetNumSlots(), gap = half / num_slots;
    std::vector<word> icrt = InverseCrtConstants(primes, degree);
    DeviceVector<word> tmp(nt * degree);
    auto g = param_.GetLimbIndices(np);
    CheckAbi(cfhe_intt(h_, tmp.data(), ptxt.mx_.data(), g.data(), nt, 1, 0, 0, icrt.data(), 0, 0));
    std::vector<word> res;
    CopyDeviceToHost(res, tmp);
    CheckAbi(cfhe_synchronize(h_));
    std::vector<detail::BigU> hat(nt);
    detail::BigU Q(1);
    Q.w[0] = 1;
    for (int j = 0; j < nt; j++) {
      Q.mul_small(primes[j]);
      hat[j] = detail::BigU(1);
      hat[j].w[0] = 1;
      for (int k = 0; k < nt; k++)
        if (k != j) hat[j].mul_small(primes[k]);
    }
    const detail::BigU halfQ = Q.half();
    auto lift = [&](int idx) {
      detail::BigU acc(Q.w.size() + 2);
      for (int j = 0; j < nt; j++) acc.add_mul(hat[j], res[(size_t)j * degree + idx]);
      while (acc.cmp(Q) >= 0) acc.sub(Q);
      if (acc.cmp(halfQ) > 0) {
        detail::BigU d = Q;
        d.sub(acc);
        return -d.to_double();
      }
      return acc.to_double();
    };
    message.resize(num_slots);
    const double scale = ptxt.GetScale();
    for (int i = 0; i < num_slots; i++)
      message[i] = Complex(lift(i * gap) / scale, lift(i * gap + half) / scale);
    SpecialFFT(message);
  }

  // ((Q / q_i) * degree)^-1 mod q_i: what the inverse transform multiplies by before the lift
  static std::vector<word> InverseCrtConstants(const std::vector<word> &primes, int degree) {
    const int nt = primes.size();
    std::vector<word> icrt(nt);
    for (int i = 0; i < nt; i++) {
      word prod = 1;
      for (int j = 0; j < nt; j++)
        if (j != i) prod = detail::MulMod(prod, primes[j] % primes[i], primes[i]);
      prod = detail::MulMod(prod, (word)degree % primes[i], primes[i]);
      icrt[i] = detail::InvMod(prod, primes[i]);
    }
    return icrt;
  }

  void EncodeConstant(Constant<word> &constant, int level, double scale, double number,
                      int num_aux = 0) const {
    const __int128 v = (__int128)(number * scale);
    NPInfo np = param_.LevelToNP(level, num_aux);
    auto primes = param_.GetPrimeVector(np);
    constant.ModifyNP(np);
    constant.SetScale(scale);
    for (int i = 0; i < np.GetNumTotal(); i++)
      constant.cx_[i] = detail::ToMontgomery(detail::ModI128(v, primes[i]), primes[i]);
  }

 private:
  static void BitReverse(std::vector<Complex> &v) {
    const int n = v.size();
    for (int i = 1, j = 0; i < n; i++) {
      int bit = n >> 1;
      for (; j & bit; bit >>= 1) j ^= bit;
      j ^= bit;
      if (i < j) std::swap(v[i], v[j]);
    }
  }
  // The slot map of CKKS with n slots: slot j is the plaintext polynomial
  // evaluated at zeta^(5^j), zeta = exp(2 pi i / 4n), the n complex numbers
  // d[k] standing for the coefficients a[k] + i a[k + n]. Because
  // 5^j = 4 t_j + 1 (mod 4n) and j -> t_j runs over all of [0, n), evaluating
  // at every slot is three plain steps: multiply d[k] by zeta^k, take the
  // length-n DFT with kernel exp(+2 pi i t k / n), read the result at t_j.
  // The inverse map undoes them in reverse order. (Same linear map as the
  // reference's special FFT, src/core/Encode.cpp:85-133, which interleaves the
  // powers of five with the butterflies instead.)
  static std::vector<int> SlotOrder(int n) {
    std::vector<int> t(n);
    const int64_t m = 4 * (int64_t)n;
    int64_t e = 1;
    for (int j = 0; j < n; j++) {
      t[j] = (int)((e - 1) / 4);
      e = e * 5 % m;
    }
    return t;
  }
  // in-place radix-2 DFT, natural order in and out, kernel exp(+-2 pi i t k / n)
  void PlainFft(std::vector<Complex> &v, bool positive) const {
    const int n = v.size();
    BitReverse(v);
    for (int len = 2; len <= n; len <<= 1) {
      const int step = M_ / len, half = len / 2;
      for (int base = 0; base < n; base += len)
        for (int k = 0; k < half; k++) {
          const Complex w = positive ? twiddle_factors_[k * step] : std::conj(twiddle_factors_[k * step]);
          const Complex x = v[base + k], y = v[base + k + half] * w;
          v[base + k] = x + y;
          v[base + k + half] = x - y;
        }
    }
  }
  void SpecialFFT(std::vector<Complex> &d) const {
    const int n = d.size(), zeta_step = M_ / (4 * n);
    for (int k = 0; k < n; k++) d[k] *= twiddle_factors_[k * zeta_step];
    PlainFft(d, true);
    const std::vector<int> t = SlotOrder(n);
    std::vector<Complex> slots(n);
    for (int j = 0; j < n; j++) slots[j] = d[t[j]];
    d.swap(slots);
  }
  void SpecialIFFT(std::vector<Complex> &d) const {
    const int n = d.size(), zeta_step = M_ / (4 * n);
    const std::vector<int> t = SlotOrder(n);
    std::vector<Complex> y(n);
    for (int j = 0; j < n; j++) y[t[j]] = d[j];
    PlainFft(y, false);
    for (int k = 0; k < n; k++) d[k] = y[k] * std::conj(twiddle_factors_[k * zeta_step]) / (double)n;
  }
  const Parameter<word> &param_;
  cfhe_context *h_;
  const int M_;
  std::vector<Complex> twiddle_factors_;
};

// ---------------------------------------------------------------- MultiLevelCiphertext
// One message held at several levels at once (reference
// include/core/MultiLevelCiphertext.h, src/core/MultiLevelCiphertext.cpp:1-86):
// polynomial evaluation asks for the same ciphertext at whatever level an
// operand needs, and Context::AddLowerLevelsUntil fills in the missing ones by
// multiplying with the constant 1 encoded at the level's rescaling ratio and
// rescaling. The per-level constants are shared by all instances and set up by
// StaticInit (Context::Create calls it).
template <typename word>
class MultiLevelCiphertext {
  using Ct = Ciphertext<word>;

 public:
  static void StaticInit(const Parameter<word> &param, const Encoder<word> &encoder) {
    param_ = &param;
    level_down_consts_.clear();
    level_down_consts_.resize(param.max_level_ + 1);
    for (int i = 1; i <= param.max_level_; i++)
      encoder.EncodeConstant(level_down_consts_.at(i), i, param.GetRescalePrimeProd(i), 1.0);
  }
  static void StaticDestroy() {
    param_ = nullptr;
    level_down_consts_.clear();
  }
  static const Constant<word> &GetLevelDownConst(int level) { return level_down_consts_.at(level); }

  explicit MultiLevelCiphertext(Ct &&ct) {
    AssertTrue(param_ != nullptr, "MultiLevelCiphertext: StaticInit has not run");
    AssertTrue(!ct.HasRx(), "MultiLevelCiphertext: Rx is not allowed.");
    AssertTrue(ct.GetNP().num_aux_ == 0, "MultiLevelCiphertext: Aux primes are not allowed.");
    const int level = param_->NPToLevel(ct.GetNP());
    level_map_.try_emplace(level, std::move(ct));
  }
  void AllocateLevel(int level) {
    AssertTrue(!Exists(level), "AddCiphertextAtLevel: Level " + std::to_string(level) + " already exists");
    level_map_.try_emplace(level, param_->LevelToNP(level, 0));
  }
  int GetMaxLevel() const {
    AssertTrue(!level_map_.empty(), "MultiLevelCiphertext: level_map_ is empty.");
    return level_map_.rbegin()->first;
  }
  int GetMinLevel() const {
    AssertTrue(!level_map_.empty(), "MultiLevelCiphertext: level_map_ is empty.");
    return level_map_.begin()->first;
  }
  Ct &AtLevel(int level) {
    AssertTrue(Exists(level), "Level does not exist");
    return level_map_.at(level);
  }
  const Ct &AtLevel(int level) const {
    AssertTrue(Exists(level), "Level does not exist");
    return level_map_.at(level);
  }
  bool Exists(int level) const { return level_map_.find(level) != level_map_.end(); }
  void Clear() { level_map_.clear(); }

 private:
  static inline const Parameter<word> *param_ = nullptr;
  static inline std::vector<Constant<word>> level_down_consts_{};
  std::map<int, Ct> level_map_;
};

// ---------------------------------------------------------------- Context
template <typename word>
class Context : public std::enable_shared_from_this<Context<word>> {
 protected:
  using Ct = Ciphertext<word>;
  using Pt = Plaintext<word>;
  using Const = Constant<word>;
  using Evk = EvaluationKey<word>;

  explicit Context(const Parameter<word> &param, int device = 0) : param_{param} {
    std::vector<int> lc;
    for (auto &c : param.level_config_) {
      lc.push_back(c.first);
      lc.push_back(c.second);
    }
    std::vector<word> ter = param.ter_primes_;
    if (ter.empty()) ter.push_back(0);
    CheckAbi(cfhe_context_create(&h_, device, param.log_degree_, param.main_primes_.data(),
                                 param.main_primes_.size(), ter.data(), param.ter_primes_.size(),
                                 param.aux_primes_.data(), param.aux_primes_.size(), lc.data(),
                                 param.level_config_.size(), param.additional_base_.first,
                                 param.additional_base_.second));
    detail::LiveHandles().insert(h_);
    detail::CurrentHandle() = h_;
    Container<word>::SetDegree(param.degree_);
    encoder_ = std::make_unique<Encoder<word>>(param, h_);
    MultiLevelCiphertext<word>::StaticInit(param, *encoder_);
  }

 public:
  // `device`: the GPU the engine context lives on (the reference is single-device)
  static ContextPtr<word> Create(const Parameter<word> &param, int device = 0) {
    return ContextPtr<word>(new Context<word>(param, device));
  }
  Context(const Context &) = delete;
  Context &operator=(const Context &) = delete;
  virtual ~Context() {
    encoder_.reset();
    if (detail::CurrentHandle() == h_) detail::CurrentHandle() = nullptr;
    detail::LiveHandles().erase(h_);
    cfhe_context_destroy(h_);
  }

  const Parameter<word> &param_;
  cfhe_context *h_ = nullptr;  // the engine behind this context
  std::unique_ptr<Encoder<word>> encoder_;
  const Encoder<word> &encoder() const { return *encoder_; }

  void Synchronize() const { CheckAbi(cfhe_synchronize(h_)); }

  void Copy(Ct &res, const Ct &a) const {
    if (&res == &a) return;
    MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale());
    NPInfo np = a.GetNP();
    ConstCt(0, res, {a.bx_.data(), a.ax_.data(), a.rx_.data()}, {nullptr, nullptr, nullptr},
            std::vector<word>(np.GetNumTotal(), 0), np, a.HasRx());  // a + 0: device copy on the stream
  }

  void Add(Ct &res, const Ct &a, const Ct &b) const { AddSub(res, a, b, 0); }
  void Sub(Ct &res, const Ct &a, const Ct &b) const { AddSub(res, a, b, 1); }
  void Add(Ct &res, const Ct &a, const Pt &b) const { PtOp(res, a, b, 0); }
  void Sub(Ct &res, const Ct &a, const Pt &b) const { PtOp(res, a, b, 1); }
  void Add(Ct &res, const Ct &a, const Const &b) const { ConstOp(res, a, b, 0); }
  void Sub(Ct &res, const Ct &a, const Const &b) const { ConstOp(res, a, b, 1); }
  void Sub(Ct &res, const Pt &a, const Ct &b) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    MatchResultWith(res, b);
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale());
    NPInfo np = res.GetNP();
    Binary(1, res.bx_.data(), a.mx_.data(), b.bx_.data(), np);
    Binary(2, res.ax_.data(), b.ax_.data(), nullptr, np);
    if (b.HasRx()) Binary(2, res.rx_.data(), b.rx_.data(), nullptr, np);
  }
  void Sub(Ct &res, const Const &a, const Ct &b) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    MatchResultWith(res, b);
    res.SetNumSlots(b.GetNumSlots());
    res.SetScale(a.GetScale());
    NPInfo np = res.GetNP();
    ConstKernel(2, res.bx_.data(), b.bx_.data(), nullptr, a.cx_, np);
    Binary(2, res.ax_.data(), b.ax_.data(), nullptr, np);
    if (b.HasRx()) Binary(2, res.rx_.data(), b.rx_.data(), nullptr, np);
  }
  void Neg(Ct &res, const Ct &a) const {
    MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale());
    NPInfo np = res.GetNP();
    BinaryCt(2, res, {a.bx_.data(), a.ax_.data(), a.rx_.data()}, {nullptr, nullptr, nullptr}, np, a.HasRx());
  }

  void Mult(Ct &res, const Ct &a, const Ct &b) const {
    AssertSameNP(a, b);
    AssertFalse(a.HasRx() || b.HasRx(), "Relinearization required before Mult Ct x Ct");
    AssertTrue(&res != &a && &res != &b, "Mult Ct x Ct: result must not alias an operand");
    res.ModifyNP(a.GetNP());
    res.PrepareRx();
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale() * b.GetScale());
    auto g = param_.GetLimbIndices(res.GetNP());
    CheckAbi(cfhe_tensor(h_, res.bx_.data(), res.ax_.data(), res.rx_.data(), a.bx_.data(),
                         a.ax_.data(), b.bx_.data(), b.ax_.data(), g.data(), g.size()));
  }
  void Mult(Ct &res, const Ct &a, const Pt &b) const {
    AssertSameNP(a, b);
    MatchResultWith(res, a);
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale() * b.GetScale());
    NPInfo np = res.GetNP();
    BinaryCt(3, res, {a.bx_.data(), a.ax_.data(), a.rx_.data()}, {b.mx_.data(), b.mx_.data(), b.mx_.data()}, np,
             a.HasRx());
  }
  void Mult(Ct &res, const Ct &a, const Const &b) const {
    AssertSameNP(a, b);
    MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale() * b.GetScale());
    NPInfo np = res.GetNP();
    ConstCt(3, res, {a.bx_.data(), a.ax_.data(), a.rx_.data()}, {nullptr, nullptr, nullptr}, b.cx_, np, a.HasRx());
  }

  // ---- products whose operands may sit at a higher level than the result:
  // the limbs of `level` are read in place out of the larger operand
  // (reference MultUnsafe / MadUnsafe, src/core/Context.cpp:357-489, 872-913).
  bool IsMultUnsafeCompatible(int level1, int level2) const {
    if (level1 == level2) return true;
    return param_.LevelToNP(Min(level1, level2)).IsSubsetOf(param_.LevelToNP(Max(level1, level2)));
  }
  void MultUnsafe(Ct &res, const Ct &a, const Ct &b, int level = -1) const {
    AssertFalse(a.HasRx() || b.HasRx(), "Relinearization required before MultUnsafe Ct x Ct");
    const NPInfo a_np = a.GetNP(), b_np = b.GetNP();
    AssertTrue(a_np.num_aux_ == 0 && b_np.num_aux_ == 0,
               "MultUnsafe Ct x Ct should be only used for ciphertexts without aux primes");
    if (level == -1) level = Min(param_.NPToLevel(a_np), param_.NPToLevel(b_np));
    if (&res == &a || &res == &b) {
      Ct tmp;
      MultUnsafe(tmp, a, b, level);
      res = std::move(tmp);
      return;
    }
    const NPInfo np = param_.LevelToNP(level, 0);
    AssertTrue(np.IsSubsetOf(a_np) && np.IsSubsetOf(b_np), "Incompatible levels for MultUnsafe Ct x Ct");
    res.ModifyNP(np);
    res.PrepareRx();
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale() * b.GetScale());
    const size_t ao = FrontIgnore(a_np, np), bo = FrontIgnore(b_np, np);
    auto g = param_.GetLimbIndices(np);
    CheckAbi(cfhe_tensor(h_, res.bx_.data(), res.ax_.data(), res.rx_.data(), a.bx_.data() + ao,
                         a.ax_.data() + ao, b.bx_.data() + bo, b.ax_.data() + bo, g.data(), g.size()));
  }
  // res = sum_t a[t] * b[t] as ONE unrelinearised three-part product (all
  // operands on the same level, without aux primes): one pass over the
  // operands instead of a MultUnsafe and an Add per term. The reference has no
  // n-ary tensor product; the words equal those of that composition.
  void MultSumUnsafe(Ct &res, const std::vector<const Ct *> &a, const std::vector<const Ct *> &b) const {
    AssertTrue(!a.empty() && a.size() == b.size(), "MultSumUnsafe: bad operand lists");
    const NPInfo np = a[0]->GetNP();
    AssertTrue(np.num_aux_ == 0, "MultSumUnsafe should be only used for ciphertexts without aux primes");
    int slots = 0;
    for (size_t t = 0; t < a.size(); t++) {
      AssertFalse(a[t]->HasRx() || b[t]->HasRx(), "Relinearization required before MultSumUnsafe");
      AssertTrue(a[t]->GetNP() == np && b[t]->GetNP() == np, "MultSumUnsafe: operands on different levels");
      AssertTrue(&res != a[t] && &res != b[t], "MultSumUnsafe cannot run in place");
      AssertSameScale(a[t]->GetScale() * b[t]->GetScale(), a[0]->GetScale() * b[0]->GetScale());
      slots = Max(slots, Max(a[t]->GetNumSlots(), b[t]->GetNumSlots()));
    }
    res.ModifyNP(np);
    res.PrepareRx();
    res.SetNumSlots(slots);
    res.SetScale(a[0]->GetScale() * b[0]->GetScale());
    auto g = param_.GetLimbIndices(np);
    constexpr size_t kChunk = 16;
    for (size_t t0 = 0; t0 < a.size(); t0 += kChunk) {
      const size_t n = Min(kChunk, a.size() - t0);
      std::vector<const word *> b1(n), a1(n), b2(n), a2(n);
      for (size_t t = 0; t < n; t++) {
        b1[t] = a[t0 + t]->bx_.data();
        a1[t] = a[t0 + t]->ax_.data();
        b2[t] = b[t0 + t]->bx_.data();
        a2[t] = b[t0 + t]->ax_.data();
      }
      CheckAbi(cfhe_tensor_accum(h_, res.bx_.data(), res.ax_.data(), res.rx_.data(), (int)n, b1.data(), a1.data(),
                                 b2.data(), a2.data(), t0 > 0, g.data(), g.size()));
    }
  }
  void MultUnsafe(Ct &res, const Ct &a, const Pt &b, int level = -1) const {
    const NPInfo a_np = a.GetNP(), b_np = b.GetNP();
    if (level == -1) level = Min(param_.NPToLevel(a_np), param_.NPToLevel(b_np));
    if (&res == &a && param_.NPToLevel(a_np) != level) {
      Ct tmp;
      MultUnsafe(tmp, a, b, level);
      res = std::move(tmp);
      return;
    }
    const NPInfo np = param_.LevelToNP(level, Min(a_np.num_aux_, b_np.num_aux_));
    AssertTrue(np.IsSubsetOf(a_np) && np.IsSubsetOf(b_np), "Incompatible levels for MultUnsafe Ct x Pt");
    AssertTrue(np.num_aux_ == 0 || (a_np.num_main_ == np.num_main_ && b_np.num_main_ == np.num_main_),
               "MultUnsafe with aux primes needs operands with the result's main primes");
    PrepareResult(res, np, a.HasRx());
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale() * b.GetScale());
    const size_t ao = FrontIgnore(a_np, np), bo = FrontIgnore(b_np, np);
    BinaryCt(3, res, {a.bx_.data() + ao, a.ax_.data() + ao, a.HasRx() ? a.rx_.data() + ao : nullptr},
             {b.mx_.data() + bo, b.mx_.data() + bo, b.mx_.data() + bo}, np, a.HasRx());
  }
  void MultUnsafe(Ct &res, const Ct &a, const Const &b, int level = -1) const {
    const NPInfo a_np = a.GetNP(), b_np = b.GetNP();
    if (level == -1) level = Min(param_.NPToLevel(a_np), param_.NPToLevel(b_np));
    if (&res == &a && param_.NPToLevel(a_np) != level) {
      Ct tmp;
      MultUnsafe(tmp, a, b, level);
      res = std::move(tmp);
      return;
    }
    const NPInfo np = param_.LevelToNP(level, Min(a_np.num_aux_, b_np.num_aux_));
    AssertTrue(np.IsSubsetOf(a_np) && np.IsSubsetOf(b_np), "Incompatible levels for MultUnsafe Ct x Const");
    AssertTrue(np.num_aux_ == 0 || a_np.num_main_ == np.num_main_,
               "MultUnsafe with aux primes needs operands with the result's main primes");
    PrepareResult(res, np, a.HasRx());
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale() * b.GetScale());
    const size_t ao = FrontIgnore(a_np, np);
    const std::vector<word> k = ConstLimbs(b, np);
    ConstCt(3, res, {a.bx_.data() + ao, a.ax_.data() + ao, a.HasRx() ? a.rx_.data() + ao : nullptr},
            {nullptr, nullptr, nullptr}, k, np, a.HasRx());
  }
  // res += a * b on the limbs of res
  void MadUnsafe(Ct &res, const Ct &a, const Const &b) const {
    const NPInfo a_np = a.GetNP(), b_np = b.GetNP(), np = res.GetNP();
    AssertTrue(np.IsSubsetOf(a_np) && np.IsSubsetOf(b_np), "Incompatible levels for MultUnsafe Ct x Const");
    AssertTrue(np.num_aux_ == 0 && a_np.num_aux_ == 0, "MadUnsafe should be only used for q primes");
    AssertTrue(res.GetNumSlots() == a.GetNumSlots(), "MadUnsafe should be only used for the same number of slots");
    AssertSameScale(res.GetScale(), a.GetScale() * b.GetScale());
    if (a.HasRx() && !res.HasRx()) {
      res.PrepareRx();
      CheckAbi(cfhe_binary(h_, 1, res.rx_.data(), res.bx_.data(), res.bx_.data(),
                           param_.GetLimbIndices(np).data(), np.GetNumTotal()));  // zero
    }
    const size_t ao = FrontIgnore(a_np, np);
    const std::vector<word> k = ConstLimbs(b, np);
    ConstCt(4, res, {a.bx_.data() + ao, a.ax_.data() + ao, a.HasRx() ? a.rx_.data() + ao : nullptr},
            {res.bx_.data(), res.ax_.data(), res.rx_.data()}, k, np, a.HasRx());
  }
  // Brings a ciphertext down to target_level one level at a time: multiply by
  // the constant 1 encoded at the level's scale, then rescale (reference
  // LevelDown, src/core/Context.cpp:915-928, which calls itself unoptimised).
  void LevelDown(Ct &res, const Ct &a, int target_level) const {
    Ct mult_temp, next;
    const int level = param_.NPToLevel(a.GetNP());
    AssertTrue(level >= target_level, "Invalid target level for LevelDown");
    AssertTrue(level <= param_.default_encryption_level_, "LevelDown starts at or below the default encryption level");
    const Ct *prev = &a;
    for (int i = level; i > target_level; i--) {
      Const one;
      encoder_->EncodeConstant(one, i, param_.GetScale(i), 1.0, 0);
      Mult(mult_temp, *prev, one);
      Rescale(next, mult_temp);
      prev = &next;
    }
    Copy(res, *prev);
  }

  void Permute(Ct &res, const Ct &a, int rot_dist) const {
    const int num_slots = a.GetNumSlots();
    int rot_idx = rot_dist % num_slots;
    if (rot_idx < 0) rot_idx += num_slots;
    if (rot_idx == 0) {
      Copy(res, a);
      return;
    }
    PermuteBy(res, a, cfhe_galois_for_rotation(h_, rot_idx), nullptr);
  }
  void PermuteConjugate(Ct &res, const Ct &a) const {
    PermuteBy(res, a, cfhe_galois_for_rotation(h_, -1), nullptr);
  }
  void MultImaginaryUnit(Ct &res, const Ct &a) const {
    MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale());
    auto g = param_.GetLimbIndices(res.GetNP());
    CheckAbi(cfhe_mul_imag_unit(h_, res.bx_.data(), a.bx_.data(), g.data(), g.size()));
    CheckAbi(cfhe_mul_imag_unit(h_, res.ax_.data(), a.ax_.data(), g.data(), g.size()));
    if (a.HasRx()) CheckAbi(cfhe_mul_imag_unit(h_, res.rx_.data(), a.rx_.data(), g.data(), g.size()));
  }

  void Rescale(Ct &res, const Ct &a) const {
    if (&res == &a) {
      Warn("Rescale is not adequate for in-place operations");
      Ct temp;
      Rescale(temp, a);
      res = std::move(temp);
      return;
    }
    AssertTrue(a.GetNP().num_aux_ == 0, "Rescale is not supported for ciphertexts with p primes");
    const int level = param_.NPToLevel(a.GetNP());
    AssertTrue(level > 0, "Not enough q primes to rescale");
    if (a.HasRx()) {
      res.ModifyNP(param_.LevelToNP(level - 1));
      res.PrepareRx();
    } else {
      res.RemoveRx();
      res.ModifyNP(param_.LevelToNP(level - 1));
    }
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale() / param_.GetRescalePrimeProd(level));
    // b and a in one call (the polynomials of a container are separate
    // allocations, so the strides are their distances)
    CheckAbi(cfhe_moddown(h_, level, 1, res.bx_.data(), a.bx_.data(), 2,
                          (long long)(res.ax_.data() - res.bx_.data()),
                          (long long)(a.ax_.data() - a.bx_.data())));
    if (a.HasRx()) CheckAbi(cfhe_moddown(h_, level, 1, res.rx_.data(), a.rx_.data(), 1, 0, 0));
  }

  void Relinearize(Ct &res, const Ct &a, const Evk &key) const { Relin(res, a, key, false); }
  void RelinearizeRescale(Ct &res, const Ct &a, const Evk &key) const { Relin(res, a, key, true); }

  void MultKey(Ct &res, const Ct &a, const Evk &key) const {
    if (a.HasRx()) {
      Relin(res, a, key, false);
      return;
    }
    NPInfo np = a.GetNP();
    const int level = param_.NPToLevel(np);
    Ct out(np);
    auto kb = KeyPtrs(key.bx_), ka = KeyPtrs(key.ax_);
    CheckKey(key, level);
    CheckAbi(cfhe_keyswitch(h_, level, out.bx_.data(), out.ax_.data(), a.ax_.data(), a.bx_.data(),
                            kb.data(), ka.data(), key.GetNP().num_main_));
    out.SetScale(a.GetScale());
    out.SetNumSlots(a.GetNumSlots());
    res = std::move(out);
  }

  // The key product on the extended basis, before ModDown (reference
  // include/core/Context.h:421-423, src/core/Context.cpp:649-737):
  //   a without rx:  accum = <ModUp(a.ax), key> + P * (a.bx, 0)
  //   a with rx:     accum = <ModUp(a.rx), key> + P * (a.bx, a.ax)
  // accum carries the level's Q limbs and all auxiliary limbs.
  void MultKeyNoModDown(Ct &accum, const Ct &a, const Evk &key) const {
    NPInfo np = a.GetNP();
    AssertTrue(np.num_aux_ == 0, "MultKeyNoModDown is not supported for ciphertexts with p primes");
    AssertTrue(&accum != &a, "In-place operation is not supported for MultKeyNoModDown");
    const int level = param_.NPToLevel(np), beta = cfhe_beta(h_, level);
    CheckKey(key, level);
    NPInfo ext(np.num_main_, np.num_ter_, param_.alpha_);
    const size_t ext_words = (size_t)ext.GetNumTotal() * param_.degree_;
    DeviceVector<word> mod_up(ext_words * beta);
    CheckAbi(cfhe_modup(h_, level, mod_up.data(), a.HasRx() ? a.rx_.data() : a.ax_.data()));
    Ct out(ext);
    auto kb = KeyPtrs(key.bx_), ka = KeyPtrs(key.ax_);
    CheckAbi(cfhe_evk_inner(h_, level, out.bx_.data(), out.ax_.data(), mod_up.data(), a.bx_.data(),
                            a.HasRx() ? a.ax_.data() : nullptr, kb.data(), ka.data(), key.GetNP().num_main_));
    out.SetScale(a.GetScale());
    out.SetNumSlots(a.GetNumSlots());
    accum = std::move(out);
  }

  // Fills ml_ct with every level from its lowest one down to min_level
  // (reference src/core/Context.cpp:931-949).
  void AddLowerLevelsUntil(MultiLevelCiphertext<word> &ml_ct, int min_level) const {
    if (ml_ct.Exists(min_level)) return;
    const int max_level = ml_ct.GetMaxLevel(), old_min_level = ml_ct.GetMinLevel();
    AssertTrue(min_level <= max_level && min_level >= 0,
               "AddLowerLevelsUntil: Invalid level " + std::to_string(min_level));
    Ct tmp;
    for (int i = old_min_level - 1; i >= min_level; i--) {
      ml_ct.AllocateLevel(i);
      Mult(tmp, ml_ct.AtLevel(i + 1), MultiLevelCiphertext<word>::GetLevelDownConst(i + 1));
      Rescale(ml_ct.AtLevel(i), tmp);
    }
  }

  void HRot(Ct &res, const Ct &a, const Evk &rot_key, int rot_dist) const {
    const int num_slots = a.GetNumSlots();
    rot_dist %= num_slots;
    if (rot_dist < 0) rot_dist += num_slots;
    if (rot_dist == 0) {
      Warn("HRot is not necessary");
      Copy(res, a);
      return;
    }
    Ct tmp;
    MultKey(tmp, a, rot_key);
    Permute(res, tmp, rot_dist);
  }
  void HConj(Ct &res, const Ct &a, const Evk &conj_key) const {
    Ct tmp;
    MultKey(tmp, a, conj_key);
    PermuteConjugate(res, tmp);
  }
  void HRotAdd(Ct &res, const Ct &a, const Ct &b, const Evk &rot_key, int rot_dist) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    AssertFalse(b.HasRx(), "HRotAdd: operands with rx are not supported");
    const int num_slots = Max(a.GetNumSlots(), b.GetNumSlots());
    rot_dist %= num_slots;
    if (rot_dist < 0) rot_dist += num_slots;
    if (rot_dist == 0) {
      Warn("HRotAdd is not necessary");
      Add(res, a, b);
      return;
    }
    Ct tmp;
    MultKey(tmp, a, rot_key);
    PermuteBy(res, tmp, cfhe_galois_for_rotation(h_, rot_dist), &b);
    res.SetNumSlots(num_slots);
  }
  void HConjAdd(Ct &res, const Ct &a, const Ct &b, const Evk &conj_key) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    AssertFalse(b.HasRx(), "HConjAdd: operands with rx are not supported");
    Ct tmp;
    MultKey(tmp, a, conj_key);
    PermuteBy(res, tmp, cfhe_galois_for_rotation(h_, -1), &b);
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
  }

  void HMult(Ct &res, const Ct &a, const Ct &b, const Evk &mult_key, bool rescale = true) const {
    AssertSameNP(a, b);
    AssertFalse(a.HasRx() || b.HasRx(), "Relinearization required before Mult Ct x Ct");
    NPInfo np = a.GetNP();
    const int level = param_.NPToLevel(np);
    AssertTrue(!rescale || level > 0, "Not enough q primes to rescale");
    CheckKey(mult_key, level);
    Ct out(param_.LevelToNP(rescale ? level - 1 : level));
    auto kb = KeyPtrs(mult_key.bx_), ka = KeyPtrs(mult_key.ax_);
    CheckAbi(cfhe_hmult(h_, level, out.bx_.data(), out.ax_.data(), a.bx_.data(), a.ax_.data(),
                        b.bx_.data(), b.ax_.data(), kb.data(), ka.data(),
                        mult_key.GetNP().num_main_, rescale));
    double scale = a.GetScale() * b.GetScale();
    if (rescale) scale /= param_.GetRescalePrimeProd(level);
    out.SetScale(scale);
    out.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res = std::move(out);
  }

  // Keeps only the limbs of `target_level` (the levels must be nested: every
  // prime of the target level is present in a). The scale is unchanged. This is
  // the limb-dropping half of the reference's LevelDown
  // (src/core/Context.cpp:872-949), without its scale correction.
  void DropToLevel(Ct &res, const Ct &a, int target_level) const {
    NPInfo np = a.GetNP(), tnp = param_.LevelToNP(target_level);
    AssertTrue(tnp.IsSubsetOf(np), "DropToLevel: levels are not nested");
    if (tnp == np) {
      Copy(res, a);
      return;
    }
    AssertTrue(&res != &a, "DropToLevel cannot run in place");
    const size_t off = (size_t)(np.num_ter_ - tnp.num_ter_) * param_.degree_;
    Ct out(tnp);
    if (a.HasRx()) out.PrepareRx();
    std::vector<word> zero(tnp.GetNumTotal(), 0);
    ConstKernel(0, out.bx_.data(), a.bx_.data() + off, nullptr, zero, tnp);
    ConstKernel(0, out.ax_.data(), a.ax_.data() + off, nullptr, zero, tnp);
    if (a.HasRx()) ConstKernel(0, out.rx_.data(), a.rx_.data() + off, nullptr, zero, tnp);
    out.SetScale(a.GetScale());
    out.SetNumSlots(a.GetNumSlots());
    res = std::move(out);
  }

  // Rotations of one ciphertext by several distances with a single ModUp
  // (the reference's HoistHandler baby step, src/extension/Hoist.cu:578-691).
  // keys[i] is the rotation key for rot_dists[i] (distances in (0, num_slots)).
  void HoistedRotate(std::vector<Ct> &res, const Ct &a, const std::vector<int> &rot_dists,
                     const std::vector<const Evk *> &keys) const {
    AssertFalse(a.HasRx(), "HoistedRotate: relinearize first");
    AssertTrue(rot_dists.size() == keys.size() && !rot_dists.empty(), "HoistedRotate: bad arguments");
    NPInfo np = a.GetNP();
    const int level = param_.NPToLevel(np), beta = cfhe_beta(h_, level);
    const size_t words = (size_t)np.GetNumQ() * param_.degree_;
    std::vector<const word *> kb, ka;
    for (const Evk *k : keys) {
      CheckKey(*k, level);
      AssertTrue(k->GetNP().num_main_ == keys[0]->GetNP().num_main_, "HoistedRotate: key shapes differ");
      for (int j = 0; j < beta; j++) {
        kb.push_back(k->bx_[j].data());
        ka.push_back(k->ax_[j].data());
      }
    }
    DeviceVector<word> out(2 * words * rot_dists.size());
    CheckAbi(cfhe_hoisted_rotations(h_, level, out.data(), a.bx_.data(), a.ax_.data(), rot_dists.size(),
                                    rot_dists.data(), kb.data(), ka.data(), keys[0]->GetNP().num_main_));
    res.clear();
    std::vector<word> zero(np.GetNumTotal(), 0);
    for (size_t i = 0; i < rot_dists.size(); i++) {
      res.emplace_back(np);
      ConstKernel(0, res[i].bx_.data(), out.data() + 2 * i * words, nullptr, zero, np);
      ConstKernel(0, res[i].ax_.data(), out.data() + (2 * i + 1) * words, nullptr, zero, np);
      res[i].SetScale(a.GetScale());
      res[i].SetNumSlots(a.GetNumSlots());
    }
  }

  void AssertSameScale(double s1, double s2) const {
    // relative tolerance of the reference (src/core/Context.cpp:53-60)
    AssertTrue(std::abs(s1 - s2) <= 1e-12 * std::abs(s1), "Scale mismatch");
  }

 protected:
  template <typename A, typename B>
  void AssertSameNP(const A &a, const B &b) const {
    AssertTrue(a.GetNP() == b.GetNP(), "NP mismatch");
  }
  void MatchResultWith(Ct &res, const Ct &a) const {
    if (a.HasRx()) {
      res.ModifyNP(a.GetNP());
      res.PrepareRx();
    } else {
      res.RemoveRx();
      res.ModifyNP(a.GetNP());
    }
  }
  // words to skip at the front of a polynomial of `big` to reach the limbs of `small`
  size_t FrontIgnore(const NPInfo &big, const NPInfo &small) const {
    return (size_t)(big.num_ter_ - small.num_ter_) * param_.degree_;
  }
  void PrepareResult(Ct &res, const NPInfo &np, bool rx) const {
    if (rx) {
      res.ModifyNP(np);
      res.PrepareRx();
    } else {
      res.RemoveRx();
      res.ModifyNP(np);
    }
  }
  // per-limb words of a constant restricted to the limbs of np
  std::vector<word> ConstLimbs(const Const &b, const NPInfo &np) const {
    const NPInfo b_np = b.GetNP();
    const int skip = b_np.num_ter_ - np.num_ter_;
    std::vector<word> k(b.cx_.begin() + skip, b.cx_.begin() + skip + np.GetNumQ());
    for (int a = 0; a < np.num_aux_; a++) k.push_back(b.cx_[b_np.GetNumQ() + a]);
    return k;
  }
  void D2D(DeviceVector<word> &dst, const DeviceVector<word> &src, const NPInfo &np) const {
    std::vector<word> zero(np.GetNumTotal(), 0);
    ConstKernel(0, dst.data(), src.data(), nullptr, zero, np);  // a + 0: device copy on the stream
  }
  // one launch for the two or three polynomials of a ciphertext
  void BinaryCt(int op, Ct &res, const word *const (&a)[3], const word *const (&b)[3], const NPInfo &np,
                bool rx) const {
    auto g = param_.GetLimbIndices(np);
    word *dst[3] = {res.bx_.data(), res.ax_.data(), rx ? res.rx_.data() : nullptr};
    CheckAbi(cfhe_elementwise_multi(h_, 0, op, rx ? 3 : 2, dst, a, b, nullptr, g.data(), g.size()));
  }
  void ConstCt(int op, Ct &res, const word *const (&a)[3], const word *const (&b)[3],
               const std::vector<word> &k, const NPInfo &np, bool rx) const {
    auto g = param_.GetLimbIndices(np);
    AssertTrue(k.size() == g.size(), "Constant has a different number of limbs");
    word *dst[3] = {res.bx_.data(), res.ax_.data(), rx ? res.rx_.data() : nullptr};
    CheckAbi(cfhe_elementwise_multi(h_, 1, op, rx ? 3 : 2, dst, a, b, k.data(), g.data(), g.size()));
  }
  void Binary(int op, word *dst, const word *a, const word *b, const NPInfo &np) const {
    auto g = param_.GetLimbIndices(np);
    CheckAbi(cfhe_binary(h_, op, dst, a, b, g.data(), g.size()));
  }
  void ConstKernel(int op, word *dst, const word *a, const word *b, const std::vector<word> &k,
                   const NPInfo &np) const {
    auto g = param_.GetLimbIndices(np);
    AssertTrue(k.size() == g.size(), "Constant has a different number of limbs");
    CheckAbi(cfhe_const_op(h_, op, dst, a, b, k.data(), g.data(), g.size()));
  }
  void AddSub(Ct &res, const Ct &a, const Ct &b, int op) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    NPInfo np = a.GetNP();
    if (a.HasRx() != b.HasRx()) {
      // an unrelinearised product plus an ordinary ciphertext: the third
      // polynomial passes through (negated when it is subtracted). The
      // reference requires relinearisation first; this saves one key switch
      // when several products at one level are summed.
      const Ct &x = a.HasRx() ? a : b;
      if (&res != &x) {
        res.ModifyNP(np);
        res.PrepareRx();
      }
      res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
      res.SetScale(a.GetScale());
      Binary(op, res.bx_.data(), a.bx_.data(), b.bx_.data(), np);
      Binary(op, res.ax_.data(), a.ax_.data(), b.ax_.data(), np);
      if (a.HasRx()) {
        if (&res != &a) D2D(res.rx_, a.rx_, np);
      } else if (op == 0) {
        if (&res != &b) D2D(res.rx_, b.rx_, np);
      } else {
        Binary(2, res.rx_.data(), b.rx_.data(), nullptr, np);
      }
      return;
    }
    MatchResultWith(res, a);
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale());
    BinaryCt(op, res, {a.bx_.data(), a.ax_.data(), a.rx_.data()}, {b.bx_.data(), b.ax_.data(), b.rx_.data()}, np,
             a.HasRx());
  }
  void PtOp(Ct &res, const Ct &a, const Pt &b, int op) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    const bool alias = &res == &a;
    if (!alias) MatchResultWith(res, a);
    res.SetNumSlots(Max(a.GetNumSlots(), b.GetNumSlots()));
    res.SetScale(a.GetScale());
    NPInfo np = a.GetNP();
    Binary(op, res.bx_.data(), a.bx_.data(), b.mx_.data(), np);
    if (!alias) {
      D2D(res.ax_, a.ax_, np);
      if (a.HasRx()) D2D(res.rx_, a.rx_, np);
    }
  }
  void ConstOp(Ct &res, const Ct &a, const Const &b, int op) const {
    AssertSameNP(a, b);
    AssertSameScale(a.GetScale(), b.GetScale());
    const bool alias = &res == &a;
    if (!alias) MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale());
    NPInfo np = a.GetNP();
    ConstKernel(op, res.bx_.data(), a.bx_.data(), nullptr, b.cx_, np);
    if (!alias) {
      D2D(res.ax_, a.ax_, np);
      if (a.HasRx()) D2D(res.rx_, a.rx_, np);
    }
  }
  void PermuteBy(Ct &res, const Ct &a, uint32_t galois, const Ct *add) const {
    if (&res == &a || &res == add) {  // in-place operation is not supported
      Ct tmp;
      PermuteBy(tmp, a, galois, add);
      res = std::move(tmp);
      return;
    }
    MatchResultWith(res, a);
    res.SetNumSlots(a.GetNumSlots());
    res.SetScale(a.GetScale());
    auto g = param_.GetLimbIndices(a.GetNP());
    CheckAbi(cfhe_permute(h_, res.bx_.data(), a.bx_.data(), add ? add->bx_.data() : nullptr, galois,
                          g.data(), g.size()));
    CheckAbi(cfhe_permute(h_, res.ax_.data(), a.ax_.data(), add ? add->ax_.data() : nullptr, galois,
                          g.data(), g.size()));
    if (a.HasRx())
      CheckAbi(cfhe_permute(h_, res.rx_.data(), a.rx_.data(), nullptr, galois, g.data(), g.size()));
  }
  std::vector<const word *> KeyPtrs(const std::vector<DeviceVector<word>> &v) const {
    std::vector<const word *> p;
    for (auto &d : v) p.push_back(d.data());
    return p;
  }
  void CheckKey(const Evk &key, int level) const {
    AssertTrue(key.GetBeta() >= cfhe_beta(h_, level), "Beta mismatch");
    AssertTrue(key.GetNP().num_ter_ == param_.GetMaxNumTer() && key.GetNP().num_aux_ == param_.alpha_,
               "Invalid evaluation key shape");
  }
  // Relinearisation of (b, a, r): switch r with the key, add P*(b, a), then
  // ModDown or ModDownAndRescale (reference src/core/Context.cpp:649-737).
  void Relin(Ct &res, const Ct &a, const Evk &key, bool rescale) const {
    AssertTrue(a.HasRx(), "Relinearize requires aux");
    NPInfo np = a.GetNP();
    const int level = param_.NPToLevel(np);
    AssertTrue(!rescale || level > 0, "Not enough q primes to rescale");
    CheckKey(key, level);
    const int alpha = param_.alpha_, n = param_.degree_;
    const int nq = np.GetNumQ(), ntot = nq + alpha, beta = cfhe_beta(h_, level);
    DeviceVector<word> mu((size_t)beta * ntot * n), acc((size_t)2 * ntot * n);
    auto kb = KeyPtrs(key.bx_), ka = KeyPtrs(key.ax_);
    CheckAbi(cfhe_modup(h_, level, mu.data(), a.rx_.data()));
    CheckAbi(cfhe_evk_inner(h_, level, acc.data(), acc.data() + (size_t)ntot * n, mu.data(),
                            a.bx_.data(), a.ax_.data(), kb.data(), ka.data(), key.GetNP().num_main_));
    Ct out(param_.LevelToNP(rescale ? level - 1 : level));
    // both polynomials in one call, written straight into the result's buffers
    CheckAbi(cfhe_moddown(h_, level, rescale ? 2 : 0, out.bx_.data(), acc.data(), 2,
                          (long long)(out.ax_.data() - out.bx_.data()), (long long)ntot * n));
    double scale = a.GetScale();
    if (rescale) scale /= param_.GetRescalePrimeProd(level);
    out.SetScale(scale);
    out.SetNumSlots(a.GetNumSlots());
    res = std::move(out);  // temporaries go back to the allocator's cache, reused in stream order
  }
};

// ---------------------------------------------------------------- EvkMap
template <typename word>
class EvkMap : public std::map<int, EvaluationKey<word>> {
 public:
  // indices of the non-rotation keys (reference include/core/EvkMap.h:23-26)
  static constexpr int kMultiplicationKeyIndex = 0;
  static constexpr int kConjugationKeyIndex = -1;
  static constexpr int kDenseToSparseKeyIndex = -2;
  static constexpr int kSparseToDenseKeyIndex = -3;
  const EvaluationKey<word> &GetDenseToSparseKey() const { return this->at(kDenseToSparseKeyIndex); }
  const EvaluationKey<word> &GetSparseToDenseKey() const { return this->at(kSparseToDenseKeyIndex); }
  const EvaluationKey<word> &GetRotationKey(int r) const {
    auto it = this->find(r);
    AssertTrue(it != this->end(), "Rotation key " + std::to_string(r) + " is not prepared");
    return it->second;
  }
  const EvaluationKey<word> &GetMultiplicationKey() const { return this->at(kMultiplicationKeyIndex); }
  const EvaluationKey<word> &GetConjugationKey() const { return this->at(kConjugationKeyIndex); }
};

// rotation distance -> highest level the key must serve (reference
// include/core/EvkRequest.h)
class EvkRequest : public std::map<int, int> {
 public:
  void AddRequest(int rot_idx, int level) {
    auto it = this->find(rot_idx);
    if (it == this->end())
      this->emplace(rot_idx, level);
    else
      it->second = Max(it->second, level);
  }
};

// ---------------------------------------------------------------- UserInterface
// Client-side test code of the reference (src/UserInterface.cu): secret and
// key generation, encryption, decryption. Sampling runs on the host.
template <typename word>
class UserInterface {
  using Ct = Ciphertext<word>;
  using Pt = Plaintext<word>;
  using Evk = EvaluationKey<word>;
  using Dv = DeviceVector<word>;

 public:
  explicit UserInterface(ContextPtr<word> context) : context_{std::move(context)} {
    const auto &param = context_->param_;
    all_np_ = param.LevelToNP(param.max_level_, param.alpha_);
    all_primes_ = param.GetPrimeVector(all_np_);
    Warn("UserInterface is for testing purposes only. Do not use in production.");
    PrepareSecrets();
    PrepareBasicEvks();
  }

  void Encrypt(Ct &ctxt, const Pt &ptxt) const {
    const auto &param = context_->param_;
    NPInfo np = ptxt.GetNP();
    ctxt.RemoveRx();
    ctxt.ModifyNP(np);
    ctxt.SetScale(ptxt.GetScale());
    ctxt.SetNumSlots(ptxt.GetNumSlots());
    auto g = param.GetLimbIndices(np);
    SampleRandomPolynomial(ctxt.ax_, np);
    Dv ex;
    SampleError(ex, np);
    Dv s = SecretLimbs(main_secret_, np);
    // b = m - a*s + e in one launch (reference kernel Encrypt, src/UserInterface.cu:17-50)
    CheckAbi(cfhe_encrypt(context_->h_, ctxt.bx_.data(), ctxt.ax_.data(), s.data(), ex.data(), ptxt.mx_.data(),
                          g.data(), g.size()));
    context_->Synchronize();
  }

  void Decrypt(Pt &ptxt, const Ct &ctxt) const {
    const auto &param = context_->param_;
    NPInfo np = ctxt.GetNP();
    AssertTrue(np.num_aux_ == 0, "Decrypt: ModDown required before decryption");
    AssertTrue(!ctxt.HasRx(), "Decrypt: Rx should be removed before decryption");
    ptxt.ModifyNP(np);
    ptxt.SetScale(ctxt.GetScale());
    ptxt.SetNumSlots(ctxt.GetNumSlots());
    auto g = param.GetLimbIndices(np);
    Dv s = SecretLimbs(main_secret_, np);
    cfhe_context *h = context_->h_;
    CheckAbi(cfhe_binary(h, 3, ptxt.mx_.data(), ctxt.ax_.data(), s.data(), g.data(), g.size()));
    CheckAbi(cfhe_binary(h, 0, ptxt.mx_.data(), ptxt.mx_.data(), ctxt.bx_.data(), g.data(), g.size()));
    context_->Synchronize();
  }

  const Evk &GetRotationKey(int rot_idx) const { return evk_map_.GetRotationKey(rot_idx); }
  const Evk &GetMultiplicationKey() const { return evk_map_.GetMultiplicationKey(); }
  const Evk &GetConjugationKey() const { return evk_map_.GetConjugationKey(); }
  const EvkMap<word> &GetEvkMap() const { return evk_map_; }

  void PrepareRotationKey(int rot_idx, int max_level = -1) {
    const auto &param = context_->param_;
    if (max_level < 0) max_level = param.max_level_;
    const int half = param.degree_ / 2;
    AssertTrue(rot_idx > 0 && rot_idx < half, "Invalid rotation index " + std::to_string(rot_idx));
    if (evk_map_.find(rot_idx) != evk_map_.end()) {
      Warn("Rotation key for rotation index " + std::to_string(rot_idx) + " already prepared");
      return;
    }
    // the secret is permuted in the opposite direction (src/UserInterface.cu:303-306)
    Dv s_rot(main_secret_.size());
    auto g = param.GetLimbIndices(all_np_);
    CheckAbi(cfhe_permute(context_->h_, s_rot.data(), main_secret_.data(), nullptr,
                          cfhe_galois_for_rotation(context_->h_, half - rot_idx), g.data(), g.size()));
    PrepareEvk(rot_idx, GetNPForEvk(max_level), s_rot, main_secret_);
  }
  void UseDeviceSampling(bool on) { device_sampling_ = on; }
  void PrepareRotationKey(const EvkRequest &req) {
    for (auto &[rot, level] : req)
      if (evk_map_.find(rot) == evk_map_.end()) PrepareRotationKey(rot, level);
  }

 private:
  static constexpr double kErrorStandardDeviation = 3.2;

  // limbs of `np` taken out of a polynomial stored on every prime
  Dv SecretLimbs(const Dv &full, const NPInfo &np) const {
    const auto &param = context_->param_;
    const int n = param.degree_;
    auto g = param.GetLimbIndices(np);
    Dv out(g.size() * n);
    std::vector<word> zero(1, 0);
    for (size_t l = 0; l < g.size(); l++) {
      int gi = g[l];
      CheckAbi(cfhe_const_op(context_->h_, 0, out.data() + l * n, full.data() + (size_t)gi * n, nullptr,
                             zero.data(), &gi, 1));
    }
    return out;
  }

  void SampleTernary(Dv &dst, int hamming_weight) {
    const auto &param = context_->param_;
    const int n = param.degree_, nt = all_primes_.size();
    std::vector<int> idx(hamming_weight);
    std::vector<word> tv(hamming_weight);
    Random::SampleWithoutReplacement(idx.data(), hamming_weight, 0, n - 1);
    Random::SampleUniformWord<word>(tv.data(), hamming_weight, 0, 1);
    std::vector<word> s((size_t)nt * n, 0);
    for (int i = 0; i < nt; i++)
      for (int j = 0; j < hamming_weight; j++)
        s[(size_t)i * n + idx[j]] = (all_primes_[i] - 2) * tv[j] + 1;  // +1 or -1
    CopyHostToDevice(dst, s);
    auto g = param.GetLimbIndices(all_np_);
    CheckAbi(cfhe_ntt(context_->h_, dst.data(), dst.data(), g.data(), nt, 1, 0, 0, 1));
  }

  void PrepareSecrets() {
    const auto &param = context_->param_;
    SampleTernary(main_secret_, param.GetDenseHammingWeight());
    if (param.IsUsingSparseSecretEncapsulation()) SampleTernary(sparse_secret_, param.GetSparseHammingWeight());
  }

  void PrepareBasicEvks() {
    const auto &param = context_->param_;
    NPInfo np = GetNPForEvk(param.max_level_);
    auto g = param.GetLimbIndices(all_np_);
    Dv s2(main_secret_.size()), sc(main_secret_.size());
    CheckAbi(cfhe_binary(context_->h_, 3, s2.data(), main_secret_.data(), main_secret_.data(), g.data(),
                         g.size()));
    PrepareEvk(EvkMap<word>::kMultiplicationKeyIndex, np, main_secret_, s2);
    CheckAbi(cfhe_permute(context_->h_, sc.data(), main_secret_.data(), nullptr,
                          cfhe_galois_for_rotation(context_->h_, -1), g.data(), g.size()));
    PrepareEvk(EvkMap<word>::kConjugationKeyIndex, np, sc, main_secret_);
    if (param.IsUsingSparseSecretEncapsulation()) {
      // dense -> sparse at the lowest level; sparse -> dense at the highest,
      // with P * s_sparse on every limb of a single digit (the reference sums
      // the digits of an ordinary key, src/UserInterface.cu:341-362)
      PrepareEvk(EvkMap<word>::kDenseToSparseKeyIndex, GetNPForEvk(0), sparse_secret_, main_secret_);
      PrepareEvk(EvkMap<word>::kSparseToDenseKeyIndex, np, main_secret_, sparse_secret_, true);
    }
  }

  // digit i: b_i = e_i - a_i * s_enc, plus P * s_target on the digit's own limbs
  // (reference src/UserInterface.cu:366-458); both secrets live on every prime.
  void PrepareEvk(int key_idx, const NPInfo &np, const Dv &enc_secret, const Dv &target_secret,
                  bool single_digit = false) {
    const auto &param = context_->param_;
    const int n = param.degree_, L = param.L_;
    const int num_q = np.GetNumQ(), alpha = single_digit ? num_q : param.alpha_;
    const int beta = single_digit ? 1 : DivCeil(num_q, np.num_aux_);
    auto g = param.GetLimbIndices(np);
    cfhe_context *h = context_->h_;
    Dv s_enc = SecretLimbs(enc_secret, np), s_tgt = SecretLimbs(target_secret, np);
    std::vector<word> p_prod(num_q);
    for (int i = 0; i < num_q; i++) {
      const word q = all_primes_[g[i]];
      word pp = 1;
      for (int j = 0; j < np.num_aux_; j++) pp = detail::MulMod(pp, all_primes_[L + j] % q, q);
      p_prod[i] = detail::ToMontgomery(pp, q);
    }
    evk_map_.erase(key_idx);
    evk_map_.try_emplace(key_idx, np, beta);
    auto &evk = evk_map_.at(key_idx);
    for (int i = 0; i < beta; i++) {
      SampleRandomPolynomial(evk.ax_[i], np);
      Dv ex;
      SampleError(ex, np);
      // an encryption of zero (EncryptZero, src/UserInterface.cu:55-80) plus
      // P * s_target on the digit's own limbs (AddEvkPart, :82-108)
      CheckAbi(cfhe_encrypt(h, evk.bx_[i].data(), evk.ax_[i].data(), s_enc.data(), ex.data(), nullptr, g.data(),
                            g.size()));
      const int lo = i * alpha, hi = Min((i + 1) * alpha, num_q);
      CheckAbi(cfhe_add_evk_part(h, evk.bx_[i].data() + (size_t)lo * n, s_tgt.data() + (size_t)lo * n,
                                 p_prod.data() + lo, g.data() + lo, hi - lo));
      context_->Synchronize();
    }
  }

  // Uniform ring element and error polynomial. By default the words are
  // generated on the device (cfhe_sample_uniform / cfhe_sample_error) from a
  // 64-bit seed drawn from the host generator, so Random::Seed still fixes
  // everything; UseDeviceSampling(false) restores the reference's host
  // sampling and upload (src/UserInterface.cu:223-276).
  void SampleRandomPolynomial(Dv &poly, const NPInfo &np) const {
    const auto &param = context_->param_;
    const int n = param.degree_;
    auto g = param.GetLimbIndices(np);
    if (device_sampling_) {
      poly.resize(g.size() * n);
      CheckAbi(cfhe_sample_uniform(context_->h_, poly.data(), g.data(), g.size(), Random::Draw64(), 0));
      return;
    }
    std::vector<word> host(g.size() * n);
    for (size_t i = 0; i < g.size(); i++) Random::SampleUniformBelow(host.data() + i * n, n, all_primes_[g[i]]);
    CopyHostToDevice(poly, host);
  }

  void SampleError(Dv &poly, const NPInfo &np) const {
    const auto &param = context_->param_;
    const int n = param.degree_;
    auto g = param.GetLimbIndices(np);
    if (device_sampling_) {
      poly.resize(g.size() * n);
      CheckAbi(cfhe_sample_error(context_->h_, poly.data(), g.data(), g.size(), kErrorStandardDeviation,
                                 Random::Draw64(), 1));
    } else {
      std::vector<int> err(n);
      Random::SampleDiscreteNormal(err.data(), n, 0, kErrorStandardDeviation);
      std::vector<word> host(g.size() * n);
      for (size_t i = 0; i < g.size(); i++) {
        const word q = all_primes_[g[i]];
        for (int j = 0; j < n; j++) host[i * n + j] = err[j] < 0 ? q - (word)(-err[j]) : (word)err[j];
      }
      CopyHostToDevice(poly, host);
    }
    CheckAbi(cfhe_ntt(context_->h_, poly.data(), poly.data(), g.data(), g.size(), 1, 0, 0, 1));
  }

  NPInfo GetNPForEvk(int max_level) const {
    const auto &param = context_->param_;
    NPInfo res = param.LevelToNP(0);
    for (int i = 1; i <= max_level; i++) res.num_main_ = Max(res.num_main_, param.LevelToNP(i).num_main_);
    res.num_ter_ = param.GetMaxNumTer();
    res.num_aux_ = param.alpha_;
    return res;
  }

  ContextPtr<word> context_;
  bool device_sampling_ = true;
  NPInfo all_np_;
  std::vector<word> all_primes_;  // every prime, global order (index = limb index g)
  Dv main_secret_;                // NTT, M-form, on every prime
  Dv sparse_secret_;              // same layout; only with sparse-secret encapsulation
  EvkMap<word> evk_map_;
};

}  // namespace cheddar
