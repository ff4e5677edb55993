// Data ingestion: example records, text parsers (libsvm, adfea, terafea, the
// native dense/sparse/sparse-binary format, criteo), per-slot statistics, file
// access (plain / gzip / stdin), record io, streaming minibatch reader, and the
// column-slot reader with an on-disk cache.
// Counterparts: data/text_parser.h:9-22 (+.cc), data/info_parser.h:8-22 (+.cc),
// data/stream_reader.h:14-214, data/slot_reader.h:8-63 (+.cc), data/common.h:9-31
// (+.cc), data/proto/example.proto:2-33, util/file.h:19-125, util/filelinereader.h:16-40,
// util/recordio.h:9-77, util/split.h:9-28, util/strtonum.h:12-45,
// data/show_example.h:8-18, data/text2proto.h:4-39.
#pragma once
#include <zlib.h>
#include <regex>
#include "matrix.h"
#include "task.h"

namespace PS {

// ---------------------------------------------------------------- strings
inline std::vector<std::string> split(const std::string& s, char delim, bool skip_empty = false) {
  std::vector<std::string> out;
  std::string cur;
  for (char c : s) {
    if (c == delim) { if (!(skip_empty && cur.empty())) out.push_back(cur); cur.clear(); }
    else cur.push_back(c);
  }
  if (!(skip_empty && cur.empty())) out.push_back(cur);
  return out;
}
inline std::string join(const std::vector<std::string>& v, const std::string& delim) {
  std::string out;
  for (size_t i = 0; i < v.size(); ++i) { if (i) out += delim; out += v[i]; }
  return out;
}
// strict numeric conversions: the whole token must parse
inline bool strtofloat(const char* s, float* v) {
  if (!s || !*s) return false;
  // plain decimals ("1", "-1", "0.25", up to 9 digits in all) are most of every data file: they need no
  // locale-aware parser; anything else (exponents, inf, long mantissas) goes to strtof
  {
    const char* p = s;
    bool neg = false;
    if (*p == '-') { neg = true; ++p; } else if (*p == '+') { ++p; }
    uint32_t mant = 0;
    int digits = 0, frac = 0;
    while (*p >= '0' && *p <= '9' && digits < 9) { mant = mant * 10 + (uint32_t)(*p - '0'); ++p; ++digits; }
    if (*p == '.') {
      ++p;
      while (*p >= '0' && *p <= '9' && digits < 9) { mant = mant * 10 + (uint32_t)(*p - '0'); ++p; ++digits; ++frac; }
    }
    if (*p == '\0' && digits > 0) {
      static const double kPow10[10] = {1, 1e1, 1e2, 1e3, 1e4, 1e5, 1e6, 1e7, 1e8, 1e9};
      const double x = (double)mant / kPow10[frac];     // exact operands; the double quotient then rounds to float
      *v = (float)(neg ? -x : x);
      return true;
    }
  }
  char* end; *v = strtof(s, &end); return *end == '\0';
}
inline bool strtoi32(const char* s, int32_t* v) {
  if (!s || !*s) return false;
  char* end; long x = strtol(s, &end, 10); *v = (int32_t)x; return *end == '\0';
}
inline bool strtou64(const char* s, uint64_t* v) {
  if (!s || !*s) return false;
  // up to 19 digits cannot overflow 64 bits
  uint64_t x = 0;
  const char* p = s;
  while (*p >= '0' && *p <= '9' && p - s < 19) { x = x * 10 + (uint64_t)(*p - '0'); ++p; }
  if (*p == '\0') { *v = x; return true; }
  char* end; *v = strtoull(s, &end, 10); return *end == '\0';
}

// ---------------------------------------------------------------- example
struct Slot {
  int id = 0;                 // 0 = label
  std::vector<uint64_t> key;
  std::vector<float> val;
};
struct Example {
  std::vector<Slot> slot;
  void Clear() { slot.clear(); }
  Slot* add_slot(int id) { slot.emplace_back(); slot.back().id = id; return &slot.back(); }
  std::string Serialize() const {
    Writer w;
    w.U64(slot.size());
    for (auto& s : slot) {
      w.I64(s.id); w.U64(s.key.size()); for (auto k : s.key) w.U64(k);
      w.U64(s.val.size()); w.Raw(s.val.data(), s.val.size() * sizeof(float));
    }
    return w.str();
  }
  bool Parse(const char* p, size_t n) {
    Reader r(p, n);
    uint64_t ns = r.U64(); slot.clear();
    for (uint64_t i = 0; i < ns && r.ok(); ++i) {
      slot.emplace_back(); Slot& s = slot.back();
      s.id = (int)r.I64();
      uint64_t nk = r.U64(); for (uint64_t j = 0; j < nk && r.ok(); ++j) s.key.push_back(r.U64());
      uint64_t nv = r.U64();
      for (uint64_t j = 0; j < nv && r.ok(); ++j) {
        uint32_t u = 0;
        for (int b = 0; b < 4; ++b) { u |= (uint32_t)r.U8() << (8 * b); }
        float f;
        memcpy(&f, &u, 4);
        s.val.push_back(f);
      }
    }
    return r.ok();
  }
  std::string ShortDebugString() const {
    std::ostringstream ss;
    for (auto& s : slot) {
      ss << "slot " << s.id << ":";
      for (size_t i = 0; i < std::max(s.key.size(), s.val.size()); ++i) {
        ss << " ";
        if (i < s.key.size()) ss << s.key[i];
        if (i < s.key.size() && i < s.val.size()) ss << ":";
        if (i < s.val.size()) ss << s.val[i];
      }
      ss << "; ";
    }
    return ss.str();
  }
};

struct SlotInfo {
  enum Format { DENSE = 1, SPARSE = 2, SPARSE_BINARY = 3 };
  Format format = SPARSE_BINARY;
  int id = 0;
  uint64_t min_key = kMaxKey, max_key = 0;
  uint64_t nnz_ele = 0, nnz_ex = 0;
};
struct ExampleInfo {
  std::vector<SlotInfo> slot;
  uint64_t num_ex = 0;
};
ExampleInfo mergeExampleInfo(const ExampleInfo& a, const ExampleInfo& b);
// matrix header of slot `i` for `num_ex` examples
MatrixInfo readMatrixInfo(const ExampleInfo& info, int slot_idx, int sizeof_idx, int sizeof_val);

// ---------------------------------------------------------------- parsers
// Reader settings that a node takes from its command line (-hash_kernel, -shuffle_fea_id, -line_limit):
// defaults of every StreamReader, ExampleParser and FileLineReader made afterwards in this process.
struct ReaderFlags {
  uint64_t hash_kernel = 0;
  bool shuffle_fea_id = false;
  int line_limit = 0;
  int parse_threads = 2;       // -num_threads: threads that parse the lines of a text minibatch
  static ReaderFlags& get() { static ReaderFlags f; return f; }
};

class ExampleParser {
 public:
  typedef DataConfig::TextFormat TextFormat;
  void Init(TextFormat format, bool ignore_fea_slot = false, bool shuffle_fea_id = false);
  // parses one line (modified in place); false if malformed
  bool ToProto(char* line, Example* ex);
 private:
  bool ParseLibsvm(char* line, Example* ex);
  bool ParseAdfea(char* line, Example* ex);
  bool ParseTerafea(char* line, Example* ex);
  bool ParsePS(char* line, Example* ex);
  bool ParseCriteo(char* line, Example* ex);
  TextFormat format_ = DataConfig::LIBSVM;
  bool ignore_fea_slot_ = false, shuffle_fea_id_ = false;
};

class InfoParser {
 public:
  bool Add(const Example& ex);
  void Clear() { for (auto& s : slot_info_) s = SlotInfo(); info_ = ExampleInfo(); num_ex_ = 0; }
  const ExampleInfo& Info();
  static const int kSlotIDmax = 4096;
 private:
  size_t num_ex_ = 0;
  ExampleInfo info_;
  SlotInfo slot_info_[kSlotIDmax];
};

// ---------------------------------------------------------------- files
// Plain, gzip (by ".gz" suffix) or stdin/stdout ("stdin"/"stdout") file; "s3://bucket/object" is read
// through a pipe from `curl` (read-only, as util/file.cc:23-61 does when built with USE_S3).
class File {
 public:
  static File* open(const std::string& name, const char* flag);
  static File* openOrDie(const std::string& name, const char* flag) {
    File* f = open(name, flag);
    PS_CHECK(f != nullptr && f->open()) << "cannot open " << name;
    return f;
  }
  static bool exists(const std::string& name);
  static bool remove(const std::string& name) { return ::remove(name.c_str()) == 0; }
  static size_t size(const std::string& name);
  ~File() { close(); }
  bool open() const { return f_ != nullptr || gz_ != nullptr; }
  size_t read(void* buf, size_t n);
  size_t write(const void* buf, size_t n);
  // one line without the trailing newline into buf (at most max-1 chars); null at EOF
  char* readLine(char* buf, int max);
  bool seek(size_t pos);
  bool flush();
  bool close();
  const std::string& filename() const { return name_; }
 private:
  File(FILE* f, gzFile gz, const std::string& name, bool std_stream, bool pipe = false)
      : f_(f), gz_(gz), name_(name), std_(std_stream), pipe_(pipe) {}
  FILE* f_ = nullptr;
  gzFile gz_ = nullptr;
  std::string name_;
  bool std_ = false;
  bool pipe_ = false;      // f_ came from popen
};
bool s3file(const std::string& name);                        // "s3://..."
std::string s3FileUrl(const std::string& name);             // http://<bucket>.s3.amazonaws.com/<object>
std::string s3DirectoryUrl(const std::string& name);        // bucket listing restricted to the prefix
bool readFileToString(const std::string& name, std::string* out);
bool writeStringToFile(const std::string& data, const std::string& name);
std::vector<std::string> readFilenamesInDirectory(const std::string& dir);
bool dirExists(const std::string& dir);
bool createDir(const std::string& dir);
std::string getPath(const std::string& full);      // directory part
std::string getFilename(const std::string& full);  // file part
std::string removeExtension(const std::string& file);
// Files in HDFS are named "hdfs://[namenode]/path" and are read through a pipe from `hadoop fs -cat`
// (util/file.cc:91-112); directories are listed with `hadoop fs -ls` (util/file.cc:350-373).
bool hdfsfile(const std::string& name);
// The command prefix "<home>/bin/hadoop fs [-D fs.default.name=..] [-D hadoop.job.ugi=..]"; an empty home
// means $HADOOP_HOME, else `hadoop` from the PATH (util/file.cc:296-302).
std::string hadoopFS(const HDFSConfig& conf);
// The prefix that File::open and the directory listing use for hdfs:// names; searchFiles sets it from a
// DataConfig that has an `hdfs` block. One setting per process, as the job has one file system.
void setHadoopFS(const HDFSConfig& conf);
std::string currentHadoopFS();
std::vector<std::string> readFilenamesInHdfsDirectory(const std::string& dir);   // full names, files only

class FileLineReader {
 public:
  explicit FileLineReader(const std::string& file, int line_limit = 0)
      : file_(file), line_limit_(line_limit > 0 ? line_limit : ReaderFlags::get().line_limit) {}
  void set_line_callback(std::function<void(char*)> cb) { cb_ = std::move(cb); }
  // calls the callback once per line
  void Reload();
  bool loaded_successfully() const { return ok_; }
 private:
  static const int kMaxLineLength = 60 * 1024;
  std::string file_;
  int line_limit_;
  bool ok_ = false;
  std::function<void(char*)> cb_;
};

// record = magic (0x3ed7230a) | u32 size | payload
class RecordWriter {
 public:
  static const uint32_t kMagicNumber = 0x3ed7230a;
  explicit RecordWriter(File* f) : file_(f) {}
  bool WriteRecord(const std::string& payload) {
    uint32_t head[2] = {kMagicNumber, (uint32_t)payload.size()};
    return file_->write(head, sizeof(head)) == sizeof(head) && file_->write(payload.data(), payload.size()) == payload.size();
  }
  template <class P> bool WriteProtocolMessage(const P& m) { return WriteRecord(m.Serialize()); }
  bool Close() { return file_->close(); }
 private:
  File* file_;
};
class RecordReader {
 public:
  explicit RecordReader(File* f) : file_(f) {}
  bool ReadRecord(std::string* payload) {
    uint32_t head[2];
    if (file_->read(head, sizeof(head)) != sizeof(head) || head[0] != RecordWriter::kMagicNumber) return false;
    payload->resize(head[1]);
    return file_->read(&(*payload)[0], head[1]) == head[1];
  }
  template <class P> bool ReadProtocolMessage(P* m) { std::string s; return ReadRecord(&s) && m->Parse(s.data(), s.size()); }
  bool Close() { return file_->close(); }
 private:
  File* file_;
};

// ---------------------------------------------------------------- file lists
// expands entries of `config.file` that are regular expressions over a directory listing
DataConfig searchFiles(const DataConfig& config);
// i-th of n parts of the file list
std::vector<DataConfig> divideFiles(const DataConfig& data, int num);
DataConfig shuffleFiles(const DataConfig& data);
DataConfig ithFile(const DataConfig& conf, int i, const std::string& suffix = "");
DataConfig appendFiles(const DataConfig& conf, const std::string& suffix);

// ---------------------------------------------------------------- stream reader
// Reads examples in chunks and assembles one matrix per slot: slot 0 (label) as
// a dense vector, every other slot as a CSR matrix with uint64 column ids.
template <typename V>
class StreamReader {
 public:
  StreamReader() {}
  explicit StreamReader(const DataConfig& data) { init(data); }
  void init(const DataConfig& data);
  void set_hash_kernel(uint64_t modulo) { hash_kernel_ = modulo; }
  // Text files: the lines of a minibatch are parsed by this many threads (the order of the examples is kept).
  void set_parse_threads(int n) { parse_threads_ = std::max(1, n); }
  // reads up to num_examples; returns false when no example was read
  bool readMatrices(uint32_t num_examples, SArray<V>* label, std::vector<std::shared_ptr<SparseMatrix<uint64_t, V>>>* mats,
                    std::vector<Example>* examples = nullptr);
  bool readExamples(uint32_t num_examples, std::vector<Example>* examples) {
    return readMatrices(num_examples, nullptr, nullptr, examples);
  }
 private:
  bool openNextFile();
  bool nextExample(Example* ex);
  DataConfig data_;
  int next_file_ = 0;
  size_t lines_in_file_ = 0;
  std::unique_ptr<File> file_;
  std::unique_ptr<RecordReader> record_;
  // format BIN: a matrix x is x.offset (uint64 row offsets), x.index (uint32 or uint64 columns), x.label
  // (float64), x.value (float32 or float64, absent for binary matrices) and the text x.info; rows are read
  // one after another from the four streams
  struct BinFiles {
    std::unique_ptr<File> offset, index, label, value;
    int sizeof_index = 4, sizeof_value = 8;
    uint64_t prev_offset = 0;
  };
  std::unique_ptr<BinFiles> bin_;
  bool openNextBin();
  bool nextBinExample(Example* ex);
  ExampleParser parser_;
  std::vector<char> line_;
  uint64_t hash_kernel_ = ReaderFlags::get().hash_kernel;
  int parse_threads_ = ReaderFlags::get().parse_threads;
  // examples parsed ahead by parseAhead(), handed out by nextExample() before it reads on
  std::vector<Example> parsed_;
  size_t parsed_pos_ = 0;
  void parseAhead(uint32_t num_examples);
};

// ---------------------------------------------------------------- slot reader
// Batch path: parses every file once into per-slot (rowsiz, colidx, value)
// arrays, caches them (compressed) on disk, and serves them from the cache on
// the next run.
class SlotReader {
 public:
  SlotReader() {}
  SlotReader(const DataConfig& data, const std::string& cache_dir) { Init(data, cache_dir); }
  void Init(const DataConfig& data, const std::string& cache_dir);
  // parses (or finds cached) all files, `num_threads` files at a time
  int Read(ExampleInfo* info = nullptr, int num_threads = 2);
  SArray<uint64_t> index(int slot_id);
  SArray<size_t> offset(int slot_id);
  SArray<float> value(int slot_id);
  void clear(int slot_id) { index_cache_.erase(slot_id); offset_cache_.erase(slot_id); }
  bool hit_cache() const { return hit_cache_; }
 private:
  std::string cacheName(const std::string& file, int slot_id) const;
  bool readOneFile(const std::string& file);
  size_t nnzEle(int slot_id) const;
  DataConfig data_;
  std::string cache_;
  ExampleInfo info_;
  std::unordered_map<int, SlotInfo> slot_info_;
  std::unordered_map<int, SArray<uint64_t>> index_cache_;
  std::unordered_map<int, SArray<size_t>> offset_cache_;
  std::mutex mu_;
  size_t loaded_file_count_ = 0;
  std::vector<uint32_t> num_ex_;
  bool hit_cache_ = false;
};

std::string showExample(const Example& ex);
// text -> record file of serialized examples; returns the number of examples written
size_t textToRecords(const DataConfig& in, const std::string& out_file);

}  // namespace PS
