// Message headers: Task (per-message header), Control (membership commands),
// Node (a participant), FilterConfig, and the application payloads, with a
// compact binary wire encoding. These are plain C++ mirrors of the reference's
// protobuf IDL: system/proto/task.proto:10-91, system/proto/node.proto:4-21,
// filter/proto/filter.proto:3-35, parameter/proto/param.proto:4-48,
// learner/proto/sgd.proto:5-26, learner/proto/bcd.proto:8-95,
// learner/proto/workload.proto:4-22.
#pragma once
#include "common.h"
#include "range.h"

namespace PS {

// ---------------------------------------------------------------- wire encoding
class Writer {
 public:
  void U8(uint8_t v) { buf_.push_back((char)v); }
  void Bool(bool v) { U8(v ? 1 : 0); }
  void U64(uint64_t v) {  // LEB128
    while (v >= 0x80) { buf_.push_back((char)(v | 0x80)); v >>= 7; }
    buf_.push_back((char)v);
  }
  void I64(int64_t v) { U64(((uint64_t)v << 1) ^ (uint64_t)(v >> 63)); }
  void F64(double v) { uint64_t u; memcpy(&u, &v, 8); Raw(&u, 8); }
  void Str(const std::string& s) { U64(s.size()); Raw(s.data(), s.size()); }
  void Raw(const void* p, size_t n) { buf_.append((const char*)p, n); }
  const std::string& str() const { return buf_; }
 private:
  std::string buf_;
};

class Reader {
 public:
  Reader(const char* p, size_t n) : p_(p), e_(p + n) {}
  bool ok() const { return ok_; }
  uint8_t U8() { if (p_ >= e_) { ok_ = false; return 0; } return (uint8_t)*p_++; }
  bool Bool() { return U8() != 0; }
  uint64_t U64() {
    uint64_t v = 0; int shift = 0;
    while (true) {
      if (p_ >= e_ || shift > 63) { ok_ = false; return 0; }
      uint8_t b = (uint8_t)*p_++;
      v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
    }
    return v;
  }
  int64_t I64() { uint64_t u = U64(); return (int64_t)(u >> 1) ^ -(int64_t)(u & 1); }
  double F64() { double v = 0; if (e_ - p_ < 8) { ok_ = false; return 0; } memcpy(&v, p_, 8); p_ += 8; return v; }
  std::string Str() {
    uint64_t n = U64();
    if ((uint64_t)(e_ - p_) < n) { ok_ = false; return ""; }
    std::string s(p_, n); p_ += n; return s;
  }
 private:
  const char* p_; const char* e_; bool ok_ = true;
};

template <typename T>
void SaveVec(Writer& w, const std::vector<T>& v) { w.U64(v.size()); for (auto& x : v) x.Save(w); }
template <typename T>
void LoadVec(Reader& r, std::vector<T>* v) {
  uint64_t n = r.U64(); v->clear();
  for (uint64_t i = 0; i < n && r.ok(); ++i) { v->emplace_back(); v->back().Load(r); }
}
inline void SaveRange(Writer& w, const Range<Key>& x) { w.U64(x.begin()); w.U64(x.end()); }
inline Range<Key> LoadRange(Reader& r) { Key b = r.U64(); Key e = r.U64(); return Range<Key>(b, e); }

// ---------------------------------------------------------------- data types
enum class DataType : uint8_t {
  OTHER = 0, INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64, FLOAT, DOUBLE, CHAR
};
template <typename V> struct TypeToEnum { static constexpr DataType v = DataType::OTHER; };
#define PS_TYPE_ENUM(T, E) template <> struct TypeToEnum<T> { static constexpr DataType v = DataType::E; }
PS_TYPE_ENUM(int8_t, INT8); PS_TYPE_ENUM(int16_t, INT16); PS_TYPE_ENUM(int32_t, INT32);
PS_TYPE_ENUM(int64_t, INT64); PS_TYPE_ENUM(uint8_t, UINT8); PS_TYPE_ENUM(uint16_t, UINT16);
PS_TYPE_ENUM(uint32_t, UINT32); PS_TYPE_ENUM(uint64_t, UINT64); PS_TYPE_ENUM(float, FLOAT);
PS_TYPE_ENUM(double, DOUBLE); PS_TYPE_ENUM(char, CHAR);
template <typename V> DataType EncodeType() { return TypeToEnum<V>::v; }

// ---------------------------------------------------------------- node
struct Node {
  enum Role { SERVER = 0, WORKER = 1, SCHEDULER = 3, GROUP = 4, UNUSED = 5 };
  Role role = UNUSED;
  std::string id;
  int rank = -1;
  std::string hostname;
  int port = 0;
  Range<Key> key = Range<Key>(0, 0);
  void Save(Writer& w) const {
    w.U8(role); w.Str(id); w.I64(rank); w.Str(hostname); w.I64(port); SaveRange(w, key);
  }
  void Load(Reader& r) {
    role = (Role)r.U8(); id = r.Str(); rank = (int)r.I64(); hostname = r.Str(); port = (int)r.I64();
    key = LoadRange(r);
  }
  std::string ShortDebugString() const {
    std::ostringstream ss;
    static const char* names[] = {"SERVER", "WORKER", "?", "SCHEDULER", "GROUP", "UNUSED"};
    ss << "role:" << names[role] << ",hostname:'" << hostname << "',port:" << port << ",id:'" << id << "'";
    if (rank >= 0) ss << ",rank:" << rank;
    return ss.str();
  }
};

struct Control {
  enum Command {
    NONE = 0,
    // a node => the scheduler
    REQUEST_APP = 1, REGISTER_NODE = 2, REPORT_PERF = 3, READY_TO_EXIT = 4,
    // the scheduler => a node
    ADD_NODE = 10, UPDATE_NODE = 11, REPLACE_NODE = 12, REMOVE_NODE = 13, EXIT = 14,
  };
  Command cmd = NONE;
  std::vector<Node> node;
  void Save(Writer& w) const { w.U8(cmd); SaveVec(w, node); }
  void Load(Reader& r) { cmd = (Command)r.U8(); LoadVec(r, &node); }
};

// ---------------------------------------------------------------- filters
struct FilterConfig {
  enum Type { KEY_CACHING = 1, COMPRESSING = 2, FIXING_FLOAT = 3, NOISE = 4 };
  struct FixedFloat {
    bool has_min = false, has_max = false;
    float min_value = -1, max_value = 1;
    void Save(Writer& w) const { w.Bool(has_min); w.Bool(has_max); w.F64(min_value); w.F64(max_value); }
    void Load(Reader& r) { has_min = r.Bool(); has_max = r.Bool(); min_value = (float)r.F64(); max_value = (float)r.F64(); }
  };
  Type type = KEY_CACHING;
  bool clear_cache_if_done = false;      // key caching
  int num_bytes = 3;                     // fixing float
  std::vector<FixedFloat> fixed_point;
  float mean = 0, std = 1;               // noise
  bool has_signature = false;            // runtime fields
  uint32_t signature = 0;
  std::vector<uint64_t> uncompressed_size;
  void Save(Writer& w) const {
    w.U8(type); w.Bool(clear_cache_if_done); w.I64(num_bytes); SaveVec(w, fixed_point);
    w.F64(mean); w.F64(std); w.Bool(has_signature); w.U64(signature);
    w.U64(uncompressed_size.size()); for (auto v : uncompressed_size) w.U64(v);
  }
  void Load(Reader& r) {
    type = (Type)r.U8(); clear_cache_if_done = r.Bool(); num_bytes = (int)r.I64(); LoadVec(r, &fixed_point);
    mean = (float)r.F64(); std = (float)r.F64(); has_signature = r.Bool(); signature = (uint32_t)r.U64();
    uint64_t n = r.U64(); uncompressed_size.clear();
    for (uint64_t i = 0; i < n && r.ok(); ++i) uncompressed_size.push_back(r.U64());
  }
};

// ---------------------------------------------------------------- parameter calls
struct TailKeyFilter {
  bool insert_count = false;
  bool has_freq_threshold = false; int freq_threshold = 0;
  bool query_value = false;
  int countmin_n = 0, countmin_k = 0;
  void Save(Writer& w) const {
    w.Bool(insert_count); w.Bool(has_freq_threshold); w.I64(freq_threshold); w.Bool(query_value);
    w.I64(countmin_n); w.I64(countmin_k);
  }
  void Load(Reader& r) {
    insert_count = r.Bool(); has_freq_threshold = r.Bool(); freq_threshold = (int)r.I64();
    query_value = r.Bool(); countmin_n = (int)r.I64(); countmin_k = (int)r.I64();
  }
};

struct ParamCall {
  bool push = true;
  int op = 0;                 // AssignOp, util/assign_op.h
  bool has_tail_filter = false;
  TailKeyFilter tail_filter;
  bool replica = false;
  void Save(Writer& w) const { w.Bool(push); w.I64(op); w.Bool(has_tail_filter); tail_filter.Save(w); w.Bool(replica); }
  void Load(Reader& r) { push = r.Bool(); op = (int)r.I64(); has_tail_filter = r.Bool(); tail_filter.Load(r); replica = r.Bool(); }
};

// ---------------------------------------------------------------- data / workload
// Where the hadoop command is and how to reach the file system (data/proto/data.proto:46-50).
struct HDFSConfig {
  std::string home;      // HADOOP_HOME
  std::string ugi;       // hadoop.job.ugi, "user,passwd"
  std::string namenode;  // fs.default.name
};

struct DataConfig {
  enum DataFormat { BIN = 1, PROTO = 2, TEXT = 3 };
  enum TextFormat { DENSE = 1, SPARSE = 2, SPARSE_BINARY = 3, ADFEA = 4, LIBSVM = 5, TERAFEA = 6, VW = 7, CRITEO = 8 };
  DataFormat format = TEXT;
  TextFormat text = LIBSVM;
  std::vector<std::string> file;
  bool ignore_feature_group = false;
  int max_num_files_per_worker = -1;
  int max_num_lines_per_file = -1;
  bool shuffle = false;
  bool has_range = false; Range<Key> range;
  int replica = 1;
  bool has_hdfs = false; HDFSConfig hdfs;   // the files are in HDFS and are read through `hadoop fs`
  void Save(Writer& w) const {
    w.U8(format); w.U8(text); w.U64(file.size()); for (auto& f : file) w.Str(f);
    w.Bool(ignore_feature_group); w.I64(max_num_files_per_worker); w.I64(max_num_lines_per_file);
    w.Bool(shuffle); w.Bool(has_range); SaveRange(w, range); w.I64(replica);
    w.Bool(has_hdfs); w.Str(hdfs.home); w.Str(hdfs.ugi); w.Str(hdfs.namenode);
  }
  void Load(Reader& r) {
    format = (DataFormat)r.U8(); text = (TextFormat)r.U8(); uint64_t n = r.U64(); file.clear();
    for (uint64_t i = 0; i < n && r.ok(); ++i) file.push_back(r.Str());
    ignore_feature_group = r.Bool(); max_num_files_per_worker = (int)r.I64();
    max_num_lines_per_file = (int)r.I64(); shuffle = r.Bool(); has_range = r.Bool();
    range = LoadRange(r); replica = (int)r.I64();
    has_hdfs = r.Bool(); hdfs.home = r.Str(); hdfs.ugi = r.Str(); hdfs.namenode = r.Str();
  }
};

struct Workload {
  enum Type { TRAIN = 1, VALIDATION = 2 };
  std::vector<int> id;
  Type type = TRAIN;
  DataConfig data;
  int replica = 1;
  bool shuffle = false;
  bool finished = false;   // the previous workload of this worker is done
  void Save(Writer& w) const {
    w.U64(id.size()); for (int i : id) w.I64(i);
    w.U8(type); data.Save(w); w.I64(replica); w.Bool(shuffle); w.Bool(finished);
  }
  void Load(Reader& r) {
    uint64_t n = r.U64(); id.clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) id.push_back((int)r.I64());
    type = (Type)r.U8(); data.Load(r); replica = (int)r.I64(); shuffle = r.Bool(); finished = r.Bool();
  }
};

struct SGDCall {
  // ROUND_LIMIT is not in the reference's sgd.proto: the scheduler of lock-step device workers grants
  // push/pull rounds in leases (round_limit = first round that may not run yet; final_round closes the job).
  enum Command { NONE = 0, REQUEST_WORKLOAD = 1, UPDATE_MODEL = 2, REPORT_PROGRESS = 3, SAVE_MODEL = 4,
                 RECOVER = 5, COMPUTE_VALIDATION_AUC = 6, ROUND_LIMIT = 7 };
  Command cmd = NONE;
  bool has_load = false;
  Workload load;
  int64_t round_limit = -1;
  bool final_round = false;
  void Save(Writer& w) const { w.U8(cmd); w.Bool(has_load); load.Save(w); w.I64(round_limit); w.Bool(final_round); }
  void Load(Reader& r) {
    cmd = (Command)r.U8(); has_load = r.Bool(); load.Load(r); round_limit = r.I64(); final_round = r.Bool();
  }
};

struct BCDCall {
  enum Command { NONE = 0, LOAD_DATA = 1, PREPROCESS_DATA = 2, UPDATE_MODEL = 3, EVALUATE_PROGRESS = 4,
                 SAVE_MODEL = 5, RECOVER = 6, COMPUTE_VALIDATION_AUC = 7, REQUEST_WORKLOAD = 8 };
  Command cmd = NONE;
  bool has_key = false; Range<Key> key;     // feature block
  int feature_group_id = 0;
  std::vector<int> fea_grp;                 // groups to preprocess
  bool hit_cache = false;
  int time = 0;                             // model-customer timestamp of this step
  int iter = 0;
  double kkt_filter_threshold = 0;
  bool reset_kkt_filter = false;
  double delta = 0;                         // tail-feature frequency etc.
  int tail_feature_freq = 0;
  void Save(Writer& w) const {
    w.U8(cmd); w.Bool(has_key); SaveRange(w, key); w.I64(feature_group_id);
    w.U64(fea_grp.size()); for (int g : fea_grp) w.I64(g);
    w.Bool(hit_cache); w.I64(time); w.I64(iter); w.F64(kkt_filter_threshold); w.Bool(reset_kkt_filter);
    w.F64(delta); w.I64(tail_feature_freq);
  }
  void Load(Reader& r) {
    cmd = (Command)r.U8(); has_key = r.Bool(); key = LoadRange(r); feature_group_id = (int)r.I64();
    uint64_t n = r.U64(); fea_grp.clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) fea_grp.push_back((int)r.I64());
    hit_cache = r.Bool(); time = (int)r.I64(); iter = (int)r.I64(); kkt_filter_threshold = r.F64();
    reset_kkt_filter = r.Bool(); delta = r.F64(); tail_feature_freq = (int)r.I64();
  }
};

// ---------------------------------------------------------------- task
struct Task {
  bool control = false;        // system control task (see ctrl) or a customer task
  bool request = false;        // request or response
  int customer_id = -1;
  bool has_time = false;
  int time = -1;               // timestamp, unique per (customer, sender)
  std::vector<int> wait_time;  // executed only after these timestamps of the same sender are finished
  bool has_key_range = false;
  Range<Key> key_range;
  int key_channel = 0;
  bool has_key = false;
  DataType key_type = DataType::OTHER;
  std::vector<DataType> value_type;
  std::vector<FilterConfig> filter;
  bool more = false;           // more header-only tasks follow: pack them into one wire message
  std::vector<Task> task;      // packed tasks
  std::string msg;             // free-form payload
  bool has_ctrl = false;  Control ctrl;
  bool has_param = false; ParamCall param;
  bool has_sgd = false;   SGDCall sgd;
  bool has_bcd = false;   BCDCall bcd;

  void set_time(int t) { time = t; has_time = true; }
  void set_key_range(const Range<Key>& r) { key_range = r; has_key_range = true; }
  ParamCall* mutable_param() { has_param = true; return &param; }
  SGDCall* mutable_sgd() { has_sgd = true; return &sgd; }
  BCDCall* mutable_bcd() { has_bcd = true; return &bcd; }
  Control* mutable_ctrl() { has_ctrl = true; return &ctrl; }

  void Save(Writer& w) const {
    uint32_t flags = (control ? 1 : 0) | (request ? 2 : 0) | (has_time ? 4 : 0) | (has_key_range ? 8 : 0) |
                     (has_key ? 16 : 0) | (more ? 32 : 0) | (has_ctrl ? 64 : 0) | (has_param ? 128 : 0) |
                     (has_sgd ? 256 : 0) | (has_bcd ? 512 : 0);
    w.U64(flags); w.I64(customer_id); w.I64(time);
    w.U64(wait_time.size()); for (int t : wait_time) w.I64(t);
    SaveRange(w, key_range); w.I64(key_channel); w.U8((uint8_t)key_type);
    w.U64(value_type.size()); for (auto t : value_type) w.U8((uint8_t)t);
    SaveVec(w, filter); SaveVec(w, task); w.Str(msg);
    if (has_ctrl) ctrl.Save(w);
    if (has_param) param.Save(w);
    if (has_sgd) sgd.Save(w);
    if (has_bcd) bcd.Save(w);
  }
  void Load(Reader& r) {
    uint32_t flags = (uint32_t)r.U64();
    control = flags & 1; request = flags & 2; has_time = flags & 4; has_key_range = flags & 8;
    has_key = flags & 16; more = flags & 32; has_ctrl = flags & 64; has_param = flags & 128;
    has_sgd = flags & 256; has_bcd = flags & 512;
    customer_id = (int)r.I64(); time = (int)r.I64();
    uint64_t n = r.U64(); wait_time.clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) wait_time.push_back((int)r.I64());
    key_range = LoadRange(r); key_channel = (int)r.I64(); key_type = (DataType)r.U8();
    n = r.U64(); value_type.clear(); for (uint64_t i = 0; i < n && r.ok(); ++i) value_type.push_back((DataType)r.U8());
    LoadVec(r, &filter); LoadVec(r, &task); msg = r.Str();
    if (has_ctrl) ctrl.Load(r);
    if (has_param) param.Load(r);
    if (has_sgd) sgd.Load(r);
    if (has_bcd) bcd.Load(r);
  }
  std::string Serialize() const { Writer w; Save(w); return w.str(); }
  bool Parse(const char* p, size_t n) { Reader r(p, n); Load(r); return r.ok(); }

  std::string ShortDebugString() const {
    std::ostringstream ss;
    ss << (control ? "ctrl " : "") << (request ? "req" : "resp") << " cust=" << customer_id << " t=" << time;
    if (!wait_time.empty()) { ss << " wait={"; for (int t : wait_time) ss << t << " "; ss << "}"; }
    if (has_key_range) ss << " kr=" << key_range;
    ss << " chl=" << key_channel;
    if (has_ctrl) ss << " cmd=" << ctrl.cmd << " nodes=" << ctrl.node.size();
    if (has_param) ss << (param.push ? " push" : " pull");
    if (has_sgd) ss << " sgd=" << sgd.cmd;
    if (has_bcd) ss << " bcd=" << bcd.cmd;
    if (more) ss << " more";
    if (!task.empty()) ss << " packed=" << task.size();
    return ss.str();
  }
};

}  // namespace PS
