#include "data.h"

#include <dirent.h>
#include <sys/stat.h>
#include <unistd.h>

#include "hash.h"

namespace PS {

// ================================================================ tokenizer
namespace {
// Splits `s` in place at any character of `delims`; empty tokens are skipped.
class Tokens {
 public:
  Tokens(char* s, const char* delims) : p_(s), delims_(delims) {}
  char* next() {
    while (*p_ && strchr(delims_, *p_)) ++p_;
    if (!*p_) return nullptr;
    char* tok = p_;
    while (*p_ && !strchr(delims_, *p_)) ++p_;
    if (*p_) { *p_ = '\0'; ++p_; }
    return tok;
  }
 private:
  char* p_;
  const char* delims_;
};
}  // namespace

void ExampleParser::Init(TextFormat format, bool ignore_fea_slot, bool shuffle_fea_id) {
  format_ = format;
  ignore_fea_slot_ = ignore_fea_slot;
  shuffle_fea_id_ = shuffle_fea_id || ReaderFlags::get().shuffle_fea_id;
  PS_CHECK(format != DataConfig::VW) << "the vw text format is not supported";
}

bool ExampleParser::ToProto(char* line, Example* ex) {
  ex->Clear();
  switch (format_) {
    case DataConfig::LIBSVM: return ParseLibsvm(line, ex);
    case DataConfig::ADFEA: return ParseAdfea(line, ex);
    case DataConfig::TERAFEA: return ParseTerafea(line, ex);
    case DataConfig::CRITEO: return ParseCriteo(line, ex);
    case DataConfig::DENSE:
    case DataConfig::SPARSE:
    case DataConfig::SPARSE_BINARY: return ParsePS(line, ex);
    default: return false;
  }
}

// "label id:val id:val ..." with ascending ids
bool ExampleParser::ParseLibsvm(char* line, Example* ex) {
  Tokens tk(line, " \t\r\n");
  char* t = tk.next();
  float label;
  if (!strtofloat(t, &label)) return false;
  ex->add_slot(0)->val.push_back(label);
  Slot* fea = ex->add_slot(1);
  uint64_t last = 0;
  while ((t = tk.next()) != nullptr) {
    char* colon = strchr(t, ':');
    if (!colon) return false;
    *colon = '\0';
    uint64_t idx;
    float val;
    if (!strtou64(t, &idx) || !strtofloat(colon + 1, &val)) return false;
    if (idx < last) return false;
    last = idx;
    fea->key.push_back(idx);
    fea->val.push_back(val);
  }
  // slot pointers may have moved; nothing else to do
  return true;
}

// "line_id 1 clicked key:group key:group ..."; a group's keys are adjacent
bool ExampleParser::ParseAdfea(char* line, Example* ex) {
  Tokens tk(line, " :\t\r\n");
  ex->add_slot(0);
  int prev_group = 0;
  uint64_t key = 0;
  char* t;
  for (int i = 0; (t = tk.next()) != nullptr; ++i) {
    if (i < 2) continue;              // line id, constant 1
    if (i == 2) {
      int32_t label;
      if (!strtoi32(t, &label)) return false;
      ex->slot[0].val.push_back(label > 0 ? 1.f : -1.f);
    } else if (i % 2 == 1) {
      if (!strtou64(t, &key)) return false;
    } else {
      int32_t group = 1;
      if (!ignore_fea_slot_ && !strtoi32(t, &group)) return false;
      if (group != prev_group) { ex->add_slot(group); prev_group = group; }
      ex->slot.back().key.push_back(key);
    }
  }
  return !ex->slot[0].val.empty();
}

// "clicked line_id | u64 u64 ..."; the top 10 bits of a value are its group
bool ExampleParser::ParseTerafea(char* line, Example* ex) {
  Tokens tk(line, " \t\r\n");
  std::unordered_map<uint64_t, size_t> slot_of_group;
  ex->add_slot(0);
  slot_of_group[0] = 0;
  char* t;
  for (int i = 0; (t = tk.next()) != nullptr; ++i) {
    if (i == 0) {
      int32_t label;
      if (!strtoi32(t, &label)) return false;
      ex->slot[0].val.push_back(label > 0 ? 1.f : -1.f);
      continue;
    }
    if (i < 3) continue;              // line id and the separator
    uint64_t key;
    if (!strtou64(t, &key)) return false;
    uint64_t group = ignore_fea_slot_ ? 1 : key >> 54;
    uint64_t fea = key;               // the whole value stays the id: fewer collisions
    if (shuffle_fea_id_) {
      uint64_t h[2];
      MurmurHash3_x64_128(&fea, 8, 512927377, h);
      fea = h[0] ^ h[1];
    }
    auto it = slot_of_group.find(group);
    if (it == slot_of_group.end()) {
      it = slot_of_group.emplace(group, ex->slot.size()).first;
      ex->add_slot((int)group);
    }
    ex->slot[it->second].key.push_back(fea);
  }
  return !ex->slot[0].val.empty();
}

// "label; group fea[:val] fea[:val] ...; group ...;"
bool ExampleParser::ParsePS(char* line, Example* ex) {
  // split into ';' sections first
  std::vector<char*> sections;
  {
    Tokens tk(line, ";\r\n");
    char* t;
    while ((t = tk.next()) != nullptr) sections.push_back(t);
  }
  if (sections.empty()) return false;
  {
    Tokens tk(sections[0], " \t");
    int32_t label = 0;
    if (!strtoi32(tk.next(), &label)) return false;
    ex->add_slot(0)->val.push_back(label > 0 ? 1.f : -1.f);
  }
  bool have_feature_slot = false;
  for (size_t s = 1; s < sections.size(); ++s) {
    Tokens tk(sections[s], " :\t");
    char* t = tk.next();
    if (!t) continue;
    if (!ignore_fea_slot_) {
      int32_t group;
      if (!strtoi32(t, &group)) return false;
      ex->add_slot(group);
    } else if (!have_feature_slot) {
      ex->add_slot(1);
      have_feature_slot = true;
    }
    Slot& slot = ex->slot.back();
    for (int i = 0; (t = tk.next()) != nullptr; ++i) {
      bool is_value = format_ == DataConfig::DENSE || (format_ == DataConfig::SPARSE && i % 2 == 1);
      if (is_value) {
        float v;
        if (!strtofloat(t, &v)) return false;
        slot.val.push_back(v);
      } else {
        uint64_t k;
        if (!strtou64(t, &k)) return false;
        slot.key.push_back(k);
      }
    }
  }
  return true;
}

// tab separated: label, 13 integer features, 26 categorical features
bool ExampleParser::ParseCriteo(char* line, Example* ex) {
  std::vector<char*> col;
  for (char* p = line;;) {
    col.push_back(p);
    char* tab = strchr(p, '\t');
    if (!tab) break;
    *tab = '\0';
    p = tab + 1;
  }
  if (col.size() < 1 + 13 + 25) return false;
  if (!col.empty()) { char* nl = strpbrk(col.back(), "\r\n"); if (nl) *nl = '\0'; }
  float label;
  if (!strtofloat(col[0], &label)) return false;
  ex->add_slot(0)->val.push_back(label > 0 ? 1.f : -1.f);
  bool have_slot = false;
  for (int i = 0; i < 13; ++i) {
    int32_t cnt;
    if (!strtoi32(col[1 + i], &cnt)) continue;        // missing value
    if (!have_slot || !ignore_fea_slot_) { ex->add_slot(i + 1); have_slot = true; }
    // integer feature i gets the i-th 13th of the key space, offset by its count
    ex->slot.back().key.push_back(kMaxKey / 13 * i + cnt);
  }
  for (int i = 0; i < 26 && 14 + i < (int)col.size(); ++i) {
    char* s = col[14 + i];
    size_t n = strlen(s);
    if (n <= 4) continue;
    if (!have_slot || !ignore_fea_slot_) { ex->add_slot(i + 14); have_slot = true; }
    uint64_t h[2];
    MurmurHash3_x64_128(s, (int)n, 512927377, h);
    ex->slot.back().key.push_back(h[0] ^ h[1]);
  }
  return true;
}

// ================================================================ info
bool InfoParser::Add(const Example& ex) {
  for (const Slot& s : ex.slot) {
    if (s.id < 0 || s.id >= kSlotIDmax) return false;
    SlotInfo& si = slot_info_[s.id];
    for (uint64_t k : s.key) { si.min_key = std::min(si.min_key, k); si.max_key = std::max(si.max_key, k + 1); }
    if (!s.key.empty()) {
      si.format = s.val.empty() ? SlotInfo::SPARSE_BINARY : SlotInfo::SPARSE;
      si.nnz_ele += s.key.size();
    } else if (!s.val.empty()) {
      si.format = SlotInfo::DENSE;
      si.nnz_ele += s.val.size();
    } else continue;
    si.nnz_ex += 1;
    si.id = s.id;
  }
  ++num_ex_;
  return true;
}

const ExampleInfo& InfoParser::Info() {
  info_ = ExampleInfo();
  info_.num_ex = num_ex_;
  for (int i = 0; i < kSlotIDmax; ++i) if (slot_info_[i].nnz_ele) { slot_info_[i].id = i; info_.slot.push_back(slot_info_[i]); }
  return info_;
}

ExampleInfo mergeExampleInfo(const ExampleInfo& a, const ExampleInfo& b) {
  std::map<int, SlotInfo> slots;
  for (auto& s : a.slot) slots[s.id] = s;
  for (auto& s : b.slot) {
    auto it = slots.find(s.id);
    if (it == slots.end()) { slots[s.id] = s; continue; }
    SlotInfo& d = it->second;
    d.min_key = std::min(d.min_key, s.min_key);
    d.max_key = std::max(d.max_key, s.max_key);
    d.nnz_ele += s.nnz_ele;
    d.nnz_ex += s.nnz_ex;
  }
  ExampleInfo out;
  out.num_ex = a.num_ex + b.num_ex;
  for (auto& kv : slots) out.slot.push_back(kv.second);
  return out;
}

MatrixInfo readMatrixInfo(const ExampleInfo& info, int slot_idx, int sizeof_idx, int sizeof_val) {
  PS_CHECK_LT((size_t)slot_idx, info.slot.size());
  const SlotInfo& s = info.slot[slot_idx];
  MatrixInfo m;
  m.type = s.format == SlotInfo::DENSE ? MatrixInfo::DENSE
         : s.format == SlotInfo::SPARSE ? MatrixInfo::SPARSE : MatrixInfo::SPARSE_BINARY;
  m.row_major = true;
  m.id = s.id;
  m.row = SizeR(0, info.num_ex);
  m.col = SizeR(s.min_key == kMaxKey ? 0 : s.min_key, s.max_key);
  m.nnz = s.nnz_ele;
  m.sizeof_index = sizeof_idx;
  m.sizeof_value = sizeof_val;
  m.nnz_per_row = info.num_ex ? (double)s.nnz_ele / info.num_ex : 0;
  return m;
}

// ================================================================ files
bool s3file(const std::string& name) { return name.compare(0, 5, "s3://") == 0 && name.size() > 5; }
static std::string s3Bucket(const std::string& name) {
  const size_t slash = name.find('/', 5);
  return name.substr(5, slash == std::string::npos ? std::string::npos : slash - 5);
}
static std::string s3Object(const std::string& name) {
  const size_t slash = name.find('/', 5);
  return slash == std::string::npos ? "" : name.substr(slash + 1);
}
std::string s3FileUrl(const std::string& name) { return "http://" + s3Bucket(name) + ".s3.amazonaws.com/" + s3Object(name); }
std::string s3DirectoryUrl(const std::string& name) {
  return "http://" + s3Bucket(name) + ".s3.amazonaws.com/?prefix=" + s3Object(name);
}
// only characters that need no quoting may reach the shell
static bool shellSafe(const std::string& s) {
  for (char c : s)
    if (!(isalnum((unsigned char)c) || strchr("._-/:?=%+~,@", c))) return false;
  return true;
}

// the same for a whole command line: blanks separate its words
static bool shellSafeCommand(const std::string& s) {
  for (char c : s)
    if (!(c == ' ' || isalnum((unsigned char)c) || strchr("._-/:?=%+~,@", c))) return false;
  return true;
}

File* File::open(const std::string& name, const char* flag) {
  if (name == "stdin") return new File(stdin, nullptr, name, true);
  if (name == "stdout") return new File(stdout, nullptr, name, true);
  if (s3file(name)) {
    if (flag[0] != 'r' || !shellSafe(name)) return nullptr;   // objects are read only
    FILE* pipe = popen(("curl -s -f -X GET " + s3FileUrl(name)).c_str(), "r");
    return pipe ? new File(pipe, nullptr, name, false, true) : nullptr;
  }
  bool gz = name.size() > 3 && name.compare(name.size() - 3, 3, ".gz") == 0;
  if (hdfsfile(name)) {
    std::string cmd = currentHadoopFS() + " -cat " + name;
    if (flag[0] != 'r' || !shellSafeCommand(cmd)) return nullptr;   // read only, like the reference
    if (gz) cmd += " | gunzip";
    FILE* pipe = popen(cmd.c_str(), "r");
    return pipe ? new File(pipe, nullptr, name, false, true) : nullptr;
  }
  if (gz) {
    gzFile g = gzopen(name.c_str(), flag);
    return g ? new File(nullptr, g, name, false) : nullptr;
  }
  FILE* f = fopen(name.c_str(), flag);
  return f ? new File(f, nullptr, name, false) : nullptr;
}
bool File::exists(const std::string& name) { return access(name.c_str(), F_OK) == 0; }
size_t File::size(const std::string& name) {
  struct stat st;
  return stat(name.c_str(), &st) == 0 ? (size_t)st.st_size : 0;
}
size_t File::read(void* buf, size_t n) {
  if (gz_) { int r = gzread(gz_, buf, (unsigned)n); return r < 0 ? 0 : (size_t)r; }
  return fread(buf, 1, n, f_);
}
size_t File::write(const void* buf, size_t n) {
  if (gz_) { int r = gzwrite(gz_, buf, (unsigned)n); return r < 0 ? 0 : (size_t)r; }
  return fwrite(buf, 1, n, f_);
}
char* File::readLine(char* buf, int max) {
  char* r = gz_ ? gzgets(gz_, buf, max) : fgets(buf, max, f_);
  if (!r) return nullptr;
  size_t n = strlen(buf);
  while (n && (buf[n - 1] == '\n' || buf[n - 1] == '\r')) buf[--n] = '\0';
  return buf;
}
bool File::seek(size_t pos) {
  if (gz_) return gzseek(gz_, (z_off_t)pos, SEEK_SET) >= 0;
  return fseek(f_, (long)pos, SEEK_SET) == 0;
}
bool File::flush() { return gz_ ? gzflush(gz_, Z_FINISH) == Z_OK : fflush(f_) == 0; }
bool File::close() {
  bool ok = true;
  if (gz_) { ok = gzclose(gz_) == Z_OK; gz_ = nullptr; }
  if (f_) { if (pipe_) ok = pclose(f_) == 0; else if (!std_) ok = fclose(f_) == 0; f_ = nullptr; }
  return ok;
}
bool readFileToString(const std::string& name, std::string* out) {
  std::unique_ptr<File> f(File::open(name, "r"));
  if (!f) return false;
  out->clear();
  char buf[65536];
  size_t n;
  while ((n = f->read(buf, sizeof(buf))) > 0) out->append(buf, n);
  return true;
}
bool writeStringToFile(const std::string& data, const std::string& name) {
  std::unique_ptr<File> f(File::open(name, "w"));
  return f && f->write(data.data(), data.size()) == data.size();
}
std::vector<std::string> readFilenamesInDirectory(const std::string& dir) {
  std::vector<std::string> out;
  DIR* d = opendir(dir.c_str());
  if (!d) return out;
  while (dirent* e = readdir(d)) {
    std::string n = e->d_name;
    if (n != "." && n != "..") out.push_back(n);
  }
  closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}
bool dirExists(const std::string& dir) { struct stat st; return stat(dir.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }
bool createDir(const std::string& dir) { return mkdir(dir.c_str(), 0755) == 0 || dirExists(dir); }
std::string getPath(const std::string& full) {
  size_t p = full.find_last_of('/');
  return p == std::string::npos ? "." : full.substr(0, p);
}
std::string getFilename(const std::string& full) {
  size_t p = full.find_last_of('/');
  return p == std::string::npos ? full : full.substr(p + 1);
}
std::string removeExtension(const std::string& file) {
  size_t p = file.find_last_of('.');
  return p == std::string::npos ? file : file.substr(0, p);
}
bool hdfsfile(const std::string& name) { return name.compare(0, 7, "hdfs://") == 0 && name.size() > 7; }
std::string hadoopFS(const HDFSConfig& conf) {
  std::string home = conf.home;
  if (home.empty()) if (const char* env = getenv("HADOOP_HOME")) home = env;
  std::string cmd = home.empty() ? "hadoop fs" : home + "/bin/hadoop fs";
  if (!conf.namenode.empty()) cmd += " -D fs.default.name=" + conf.namenode;
  if (!conf.ugi.empty()) cmd += " -D hadoop.job.ugi=" + conf.ugi;
  return cmd;
}
namespace {
std::mutex hadoop_mu;
std::string hadoop_cmd;   // empty: not set, the default prefix is used
}  // namespace
void setHadoopFS(const HDFSConfig& conf) {
  std::lock_guard<std::mutex> l(hadoop_mu);
  hadoop_cmd = hadoopFS(conf);
}
std::string currentHadoopFS() {
  std::lock_guard<std::mutex> l(hadoop_mu);
  return hadoop_cmd.empty() ? hadoopFS(HDFSConfig()) : hadoop_cmd;
}
std::vector<std::string> readFilenamesInHdfsDirectory(const std::string& dir) {
  std::vector<std::string> out;
  const std::string cmd = currentHadoopFS() + " -ls " + dir;
  if (!shellSafeCommand(cmd)) return out;
  FILE* pipe = popen(cmd.c_str(), "r");
  if (!pipe) return out;
  // permissions, replication, owner, group, size, date, time, name: anything else (the "Found n items"
  // line) is skipped, and so are directories
  char line[10000];
  while (fgets(line, sizeof(line), pipe)) {
    std::vector<std::string> col;
    std::istringstream in(line);
    for (std::string w; in >> w;) col.push_back(w);
    if (col.size() != 8 || col[0][0] == 'd') continue;
    out.push_back(col.back());
  }
  pclose(pipe);
  std::sort(out.begin(), out.end());
  return out;
}

void FileLineReader::Reload() {
  std::unique_ptr<File> f(File::open(file_, "r"));
  ok_ = false;
  if (!f) return;
  std::vector<char> line(kMaxLineLength);
  int n = 0;
  while (f->readLine(line.data(), kMaxLineLength)) {
    if (cb_) cb_(line.data());
    if (line_limit_ > 0 && ++n >= line_limit_) break;
  }
  ok_ = true;
}

// ================================================================ file lists
DataConfig searchFiles(const DataConfig& config) {
  DataConfig out = config;
  out.file.clear();
  if (config.has_hdfs) setHadoopFS(config.hdfs);
  for (const std::string& given : config.file) {
    // with an `hdfs` block plain paths name HDFS files: "/a/b" becomes "hdfs:///a/b", a URI that hadoop takes
    const std::string pat = config.has_hdfs && !hdfsfile(given) ? "hdfs://" + given : given;
    if (hdfsfile(pat)) {
      const std::string dir = getPath(pat);
      std::regex re;
      try { re = std::regex(getFilename(pat)); } catch (const std::regex_error&) { continue; }
      size_t found = 0;
      for (const std::string& f : readFilenamesInHdfsDirectory(dir)) {
        if (!std::regex_match(getFilename(f), re)) continue;
        // `-ls` prints full paths, with or without the scheme
        out.file.push_back(hdfsfile(f) ? f : "hdfs://" + f);
        ++found;
      }
      if (!found) out.file.push_back(pat);      // no listing: take the name as a file
      continue;
    }
    if (File::exists(pat)) { out.file.push_back(pat); continue; }
    if (config.format == DataConfig::BIN) {
      // a binary matrix x is the files x.index, x.offset, x.label, x.info (and x.value): the pattern names x
      static const char* kSuffix[] = {".index", ".offset", ".value", ".label", ".info"};
      if (File::exists(pat + ".info")) { out.file.push_back(pat); continue; }
      const std::string dir = getPath(pat);
      std::regex re;
      try { re = std::regex(getFilename(pat)); } catch (const std::regex_error&) { continue; }
      for (std::string f : readFilenamesInDirectory(dir)) {
        for (const char* suf : kSuffix) {
          const size_t n = strlen(suf);
          if (f.size() > n && f.compare(f.size() - n, n, suf) == 0) { f.resize(f.size() - n); break; }
        }
        const std::string full = dir + "/" + f;
        if (std::regex_match(f, re) && std::find(out.file.begin(), out.file.end(), full) == out.file.end())
          out.file.push_back(full);
      }
      continue;
    }
    if (s3file(pat)) {
      // the bucket's listing for the directory part, objects whose file name matches the pattern
      const std::string dir_name = getPath(pat);
      std::regex re;
      try { re = std::regex(getFilename(pat)); } catch (const std::regex_error&) { continue; }
      std::string listing;
      if (shellSafe(dir_name)) {
        if (FILE* pipe = popen(("curl -s -f -X GET " + s3DirectoryUrl(dir_name + "/")).c_str(), "r")) {
          char buf[4096];
          size_t n;
          while ((n = fread(buf, 1, sizeof(buf), pipe)) > 0) listing.append(buf, n);
          pclose(pipe);
        }
      }
      size_t at = 0, found = 0;
      while ((at = listing.find("<Key>", at)) != std::string::npos) {
        const size_t end = listing.find("</Key>", at);
        if (end == std::string::npos) break;
        const std::string object = listing.substr(at + 5, end - at - 5);
        if (std::regex_match(getFilename(object), re)) { out.file.push_back("s3://" + s3Bucket(pat) + "/" + object); ++found; }
        at = end;
      }
      if (!found) out.file.push_back(pat);      // no listing (or nothing matched): take the name as an object
      continue;
    }
    std::string dir = getPath(pat);
    std::regex re;
    try { re = std::regex(getFilename(pat)); } catch (const std::regex_error&) { continue; }
    for (const std::string& f : readFilenamesInDirectory(dir)) {
      if (std::regex_match(f, re)) out.file.push_back(dir + "/" + f);
    }
  }
  if (config.max_num_files_per_worker >= 0 && (int)out.file.size() > config.max_num_files_per_worker)
    out.file.resize(config.max_num_files_per_worker);
  return out;
}
std::vector<DataConfig> divideFiles(const DataConfig& data, int num) {
  PS_CHECK_GT(num, 0);
  std::vector<DataConfig> parts(num, data);
  for (auto& p : parts) p.file.clear();
  size_t n = data.file.size();
  for (int i = 0; i < num; ++i) {
    SizeR r = SizeR(0, n).EvenDivide(num, i);
    for (size_t f = r.begin(); f < r.end(); ++f) parts[i].file.push_back(data.file[f]);
  }
  return parts;
}
DataConfig shuffleFiles(const DataConfig& data) {
  DataConfig out = data;
  std::mt19937 g((unsigned)time(nullptr));
  std::shuffle(out.file.begin(), out.file.end(), g);
  return out;
}
DataConfig ithFile(const DataConfig& conf, int i, const std::string& suffix) {
  PS_CHECK_LT((size_t)i, conf.file.size());
  DataConfig out = conf;
  out.file = {conf.file[i] + suffix};
  return out;
}
DataConfig appendFiles(const DataConfig& conf, const std::string& suffix) {
  DataConfig out = conf;
  for (auto& f : out.file) f += suffix;
  return out;
}

// ================================================================ stream reader
template <typename V>
void StreamReader<V>::init(const DataConfig& data) {
  data_ = searchFiles(data);
  // the process-wide -line_limit applies to text files whose configuration sets no limit of its own
  if (data_.max_num_lines_per_file < 0 && ReaderFlags::get().line_limit > 0 && data_.format == DataConfig::TEXT)
    data_.max_num_lines_per_file = ReaderFlags::get().line_limit;
  next_file_ = 0;
  file_.reset();
  record_.reset();
  bin_.reset();
  parsed_.clear();
  parsed_pos_ = 0;
  line_.resize(60 * 1024);
  if (data_.format == DataConfig::TEXT) parser_.Init(data_.text, data_.ignore_feature_group);
}

template <typename V>
bool StreamReader<V>::openNextFile() {
  while (next_file_ < (int)data_.file.size()) {
    file_.reset(File::open(data_.file[next_file_++], "r"));
    lines_in_file_ = 0;
    if (file_) {
      record_.reset(data_.format == DataConfig::PROTO ? new RecordReader(file_.get()) : nullptr);
      return true;
    }
    PS_LOG(WARN) << "cannot open " << data_.file[next_file_ - 1];
  }
  return false;
}

template <typename V>
bool StreamReader<V>::openNextBin() {
  while (next_file_ < (int)data_.file.size()) {
    const std::string name = data_.file[next_file_++];
    lines_in_file_ = 0;
    std::string info;
    auto b = std::make_unique<BinFiles>();
    if (readFileToString(name + ".info", &info)) {
      bool binary = false;
      for (const std::string& line : split(info, '\n', true)) {
        const size_t colon = line.find(':');
        if (colon == std::string::npos) continue;
        std::istringstream k(line.substr(0, colon)), v(line.substr(colon + 1));
        std::string key, val;
        k >> key; v >> val;
        if (key == "sizeof_index") b->sizeof_index = atoi(val.c_str());
        else if (key == "sizeof_value") b->sizeof_value = atoi(val.c_str());
        else if (key == "bool_value") binary = val == "true";
      }
      b->offset.reset(File::open(name + ".offset", "r"));
      b->index.reset(File::open(name + ".index", "r"));
      b->label.reset(File::open(name + ".label", "r"));
      if (!binary) b->value.reset(File::open(name + ".value", "r"));
      uint64_t first = 0;
      const bool sizes_ok = (b->sizeof_index == 4 || b->sizeof_index == 8) && (b->sizeof_value == 4 || b->sizeof_value == 8);
      if (sizes_ok && b->offset && b->index && b->label && (binary || b->value) && b->offset->read(&first, 8) == 8) {
        b->prev_offset = first;
        bin_ = std::move(b);
        return true;
      }
    }
    PS_LOG(WARN) << "cannot open the binary matrix " << name;
  }
  return false;
}

template <typename V>
bool StreamReader<V>::nextBinExample(Example* ex) {
  while (true) {
    if (!bin_ && !openNextBin()) return false;
    uint64_t next = 0;
    const bool limit = data_.max_num_lines_per_file >= 0 && (int)lines_in_file_ >= data_.max_num_lines_per_file;
    if (!limit && bin_->offset->read(&next, 8) == 8 && next >= bin_->prev_offset) {
      const size_t k = next - bin_->prev_offset;
      bin_->prev_offset = next;
      ++lines_in_file_;
      double lab = 0;
      if (bin_->label->read(&lab, 8) != 8) lab = 0;
      ex->Clear();
      ex->add_slot(0)->val.push_back((float)lab);
      Slot* fea = ex->add_slot(1);
      fea->key.resize(k);
      bool ok = true;
      if (bin_->sizeof_index == 8) {
        ok = bin_->index->read(fea->key.data(), 8 * k) == 8 * k;
      } else {
        std::vector<uint32_t> narrow(k);
        ok = bin_->index->read(narrow.data(), 4 * k) == 4 * k;
        for (size_t i = 0; i < k; ++i) fea->key[i] = narrow[i];
      }
      if (ok && bin_->value) {
        fea->val.resize(k);
        if (bin_->sizeof_value == 4) {
          ok = bin_->value->read(fea->val.data(), 4 * k) == 4 * k;
        } else {
          std::vector<double> wide(k);
          ok = bin_->value->read(wide.data(), 8 * k) == 8 * k;
          for (size_t i = 0; i < k; ++i) fea->val[i] = (float)wide[i];
        }
      }
      if (ok) return true;
      PS_LOG(WARN) << "the binary matrix " << data_.file[next_file_ - 1] << " ends inside a row";
    }
    bin_.reset();  // end of this matrix
  }
}

// Reads the lines of up to `num_examples` examples (one thread: the file is a stream) and parses them on
// parse_threads_ threads, each taking a contiguous share of the lines; parsed_ keeps their order.
template <typename V>
void StreamReader<V>::parseAhead(uint32_t num_examples) {
  parsed_.clear();
  parsed_pos_ = 0;
  std::vector<std::string> lines;
  lines.reserve(num_examples);
  while (lines.size() < num_examples) {
    if (!file_ && !openNextFile()) break;
    const bool limit = data_.max_num_lines_per_file >= 0 && (int)lines_in_file_ >= data_.max_num_lines_per_file;
    if (!limit && file_->readLine(line_.data(), (int)line_.size())) {
      ++lines_in_file_;
      lines.emplace_back(line_.data());
      continue;
    }
    file_.reset();  // end of this file
  }
  if (lines.empty()) return;
  const int T = (int)std::min<size_t>(parse_threads_, (lines.size() + 255) / 256);
  std::vector<std::vector<Example>> part(T);
  auto work = [&](int t) {
    const size_t b = lines.size() * t / T, e = lines.size() * (t + 1) / T;
    part[t].reserve(e - b);
    Example ex;
    for (size_t i = b; i < e; ++i)
      if (parser_.ToProto(&lines[i][0], &ex)) part[t].push_back(std::move(ex));
  };
  std::vector<std::thread> threads;
  for (int t = 1; t < T; ++t) threads.emplace_back(work, t);
  work(0);
  for (auto& th : threads) th.join();
  for (auto& p : part) for (auto& ex : p) parsed_.push_back(std::move(ex));
}

template <typename V>
bool StreamReader<V>::nextExample(Example* ex) {
  if (parsed_pos_ < parsed_.size()) { *ex = std::move(parsed_[parsed_pos_++]); return true; }
  if (data_.format == DataConfig::BIN) return nextBinExample(ex);
  while (true) {
    if (!file_ && !openNextFile()) return false;
    bool limit = data_.max_num_lines_per_file >= 0 && (int)lines_in_file_ >= data_.max_num_lines_per_file;
    if (!limit) {
      if (data_.format == DataConfig::TEXT) {
        bool got = false;
        while (file_->readLine(line_.data(), (int)line_.size())) {
          ++lines_in_file_;
          if (parser_.ToProto(line_.data(), ex)) { got = true; break; }
          limit = data_.max_num_lines_per_file >= 0 && (int)lines_in_file_ >= data_.max_num_lines_per_file;
          if (limit) break;
        }
        if (got) return true;
      } else if (data_.format == DataConfig::PROTO) {
        ++lines_in_file_;
        if (record_->ReadProtocolMessage(ex)) return true;
      }
    }
    file_.reset();  // end of this file
    record_.reset();
  }
}

template <typename V>
bool StreamReader<V>::readMatrices(uint32_t num_examples, SArray<V>* label,
                                   std::vector<std::shared_ptr<SparseMatrix<uint64_t, V>>>* mats,
                                   std::vector<Example>* examples) {
  struct Col { SArray<size_t> off; SArray<uint64_t> idx; SArray<V> val; bool has_val = false; };
  std::map<int, Col> cols;
  if (label) label->clear();
  if (examples) examples->clear();
  uint32_t n = 0;
  Example ex;
  if (data_.format == DataConfig::TEXT && parse_threads_ > 1 && num_examples >= 256 && parsed_pos_ >= parsed_.size())
    parseAhead(num_examples);
  while (n < num_examples && nextExample(&ex)) {
    if (examples) examples->push_back(ex);
    bool has_label = false;
    for (const Slot& s : ex.slot) {
      if (s.id == 0) { if (label && !s.val.empty()) { label->push_back((V)s.val[0]); has_label = true; } continue; }
      Col& c = cols[s.id];
      if (c.off.empty()) c.off.push_back(0);
      while (c.off.size() < (size_t)n + 1) c.off.push_back(c.off.back());  // rows without this slot
      for (size_t i = 0; i < s.key.size(); ++i) {
        uint64_t k = s.key[i];
        if (hash_kernel_) k %= hash_kernel_;
        c.idx.push_back(k);
        if (!s.val.empty()) { c.val.push_back((V)s.val[i]); c.has_val = true; }
      }
      c.off.push_back(c.idx.size());
    }
    if (label && !has_label) label->push_back(0);
    ++n;
  }
  if (n == 0) return false;
  if (mats) {
    mats->clear();
    for (auto& kv : cols) {
      Col& c = kv.second;
      if (c.off.empty()) c.off.push_back(0);
      while (c.off.size() < (size_t)n + 1) c.off.push_back(c.off.back());
      MatrixInfo info;
      info.type = c.has_val ? MatrixInfo::SPARSE : MatrixInfo::SPARSE_BINARY;
      info.row_major = true;
      info.id = kv.first;
      info.row = SizeR(0, n);
      uint64_t lo = kMaxKey, hi = 0;
      for (size_t i = 0; i < c.idx.size(); ++i) { lo = std::min(lo, c.idx[i]); hi = std::max(hi, c.idx[i] + 1); }
      info.col = SizeR(c.idx.empty() ? 0 : lo, hi);
      info.nnz = c.idx.size();
      info.sizeof_index = sizeof(uint64_t);
      info.sizeof_value = c.has_val ? sizeof(V) : 0;
      info.nnz_per_row = (double)c.idx.size() / n;
      mats->push_back(std::make_shared<SparseMatrix<uint64_t, V>>(info, c.off, c.idx, c.val));
    }
  }
  return true;
}
template class StreamReader<float>;
template class StreamReader<double>;

// ================================================================ slot reader
void SlotReader::Init(const DataConfig& data, const std::string& cache_dir) {
  data_ = searchFiles(data);
  cache_ = cache_dir;
  if (!cache_.empty()) createDir(cache_);
  info_ = ExampleInfo();
  slot_info_.clear();
  index_cache_.clear();
  offset_cache_.clear();
  num_ex_.assign(data_.file.size(), 0);
  loaded_file_count_ = 0;
}

std::string SlotReader::cacheName(const std::string& file, int slot_id) const {
  std::string base = cache_.empty() ? "/tmp" : cache_;
  std::string flat = file;
  for (auto& c : flat) if (c == '/') c = '_';
  return base + "/" + flat + "_slot_" + std::to_string(slot_id);
}

static bool writeInfo(const ExampleInfo& info, const std::string& name) {
  Writer w;
  w.U64(info.num_ex); w.U64(info.slot.size());
  for (auto& s : info.slot) { w.U8(s.format); w.I64(s.id); w.U64(s.min_key); w.U64(s.max_key); w.U64(s.nnz_ele); w.U64(s.nnz_ex); }
  return writeStringToFile(w.str(), name);
}
static bool readInfo(const std::string& name, ExampleInfo* info) {
  std::string s;
  if (!readFileToString(name, &s)) return false;
  Reader r(s.data(), s.size());
  info->num_ex = r.U64();
  uint64_t n = r.U64();
  info->slot.clear();
  for (uint64_t i = 0; i < n && r.ok(); ++i) {
    SlotInfo si;
    si.format = (SlotInfo::Format)r.U8(); si.id = (int)r.I64(); si.min_key = r.U64(); si.max_key = r.U64();
    si.nnz_ele = r.U64(); si.nnz_ex = r.U64();
    info->slot.push_back(si);
  }
  return r.ok();
}
template <typename T>
static bool writeCompressed(const SArray<T>& a, const std::string& name) {
  SArray<char> c = a.CompressTo();
  Writer w;
  w.U64(a.size());
  std::string head = w.str();
  std::unique_ptr<File> f(File::open(name, "w"));
  return f && f->write(head.data(), head.size()) == head.size() && f->write(c.data(), c.size()) == c.size();
}
template <typename T>
static bool readCompressed(const std::string& name, SArray<T>* a) {
  std::string s;
  if (!readFileToString(name, &s)) return false;
  Reader r(s.data(), s.size());
  uint64_t n = r.U64();
  if (!r.ok()) return false;
  size_t head = 0;
  { Writer w; w.U64(n); head = w.str().size(); }
  a->resize(n);
  if (n) a->UncompressFrom(s.data() + head, s.size() - head);
  return true;
}

bool SlotReader::readOneFile(const std::string& file) {
  std::string info_name = cacheName(file, 0) + ".info";
  ExampleInfo info;
  if (readInfo(info_name, &info)) {
    // the cache of this file exists
    Lock l(mu_);
    info_ = mergeExampleInfo(info_, info);
    hit_cache_ = true;
    return true;
  }
  DataConfig one = data_;
  one.file = {file};
  StreamReader<float> reader(one);
  struct Acc { SArray<uint64_t> colidx; SArray<uint16_t> rowsiz; SArray<float> value; };
  std::map<int, Acc> acc;
  InfoParser parser;
  std::vector<Example> exs;
  size_t num_ex = 0;
  while (reader.readExamples(4096, &exs)) {
    for (const Example& ex : exs) {
      parser.Add(ex);
      for (const Slot& s : ex.slot) {
        Acc& a = acc[s.id];
        while (a.rowsiz.size() < num_ex) a.rowsiz.push_back(0);
        if (s.id == 0) { for (float v : s.val) a.value.push_back(v); a.rowsiz.push_back((uint16_t)s.val.size()); continue; }
        for (uint64_t k : s.key) a.colidx.push_back(k);
        for (float v : s.val) a.value.push_back(v);
        a.rowsiz.push_back((uint16_t)std::min<size_t>(std::max(s.key.size(), s.val.size()), 65535));
      }
      ++num_ex;
    }
  }
  info = parser.Info();
  for (auto& kv : acc) {
    Acc& a = kv.second;
    while (a.rowsiz.size() < num_ex) a.rowsiz.push_back(0);
    std::string base = cacheName(file, kv.first);
    if (!writeCompressed(a.colidx, base + ".colidx") || !writeCompressed(a.rowsiz, base + ".rowsiz") ||
        !writeCompressed(a.value, base + ".value")) return false;
  }
  if (!writeInfo(info, info_name)) return false;
  Lock l(mu_);
  info_ = mergeExampleInfo(info_, info);
  return true;
}

int SlotReader::Read(ExampleInfo* info, int num_threads) {
  hit_cache_ = false;
  {
    ThreadPool pool(std::max(1, num_threads));
    for (const std::string& f : data_.file) pool.add([this, f] { if (!readOneFile(f)) PS_LOG(ERROR) << "failed to parse " << f; });
    pool.startWorkers();
  }
  for (auto& s : info_.slot) slot_info_[s.id] = s;
  if (info) *info = info_;
  return 0;
}

SArray<uint64_t> SlotReader::index(int slot_id) {
  { Lock l(mu_); auto it = index_cache_.find(slot_id); if (it != index_cache_.end()) return it->second; }
  SArray<uint64_t> all;
  for (const std::string& f : data_.file) {
    SArray<uint64_t> part;
    if (readCompressed(cacheName(f, slot_id) + ".colidx", &part)) all.append(part);
  }
  Lock l(mu_);
  index_cache_[slot_id] = all;
  return all;
}

SArray<size_t> SlotReader::offset(int slot_id) {
  { Lock l(mu_); auto it = offset_cache_.find(slot_id); if (it != offset_cache_.end()) return it->second; }
  SArray<size_t> off;
  off.push_back(0);
  for (const std::string& f : data_.file) {
    SArray<uint16_t> rowsiz;
    if (!readCompressed(cacheName(f, slot_id) + ".rowsiz", &rowsiz)) {
      // the slot does not appear in this file: its rows are empty
      ExampleInfo fi;
      if (readInfo(cacheName(f, 0) + ".info", &fi)) for (uint64_t i = 0; i < fi.num_ex; ++i) off.push_back(off.back());
      continue;
    }
    for (size_t i = 0; i < rowsiz.size(); ++i) off.push_back(off.back() + rowsiz[i]);
  }
  Lock l(mu_);
  offset_cache_[slot_id] = off;
  return off;
}

SArray<float> SlotReader::value(int slot_id) {
  SArray<float> all;
  for (const std::string& f : data_.file) {
    SArray<float> part;
    if (readCompressed(cacheName(f, slot_id) + ".value", &part)) all.append(part);
  }
  return all;
}

std::string showExample(const Example& ex) { return ex.ShortDebugString(); }

size_t textToRecords(const DataConfig& in, const std::string& out_file) {
  StreamReader<float> reader(in);
  std::unique_ptr<File> f(File::openOrDie(out_file, "w"));
  RecordWriter w(f.get());
  std::vector<Example> exs;
  size_t n = 0;
  while (reader.readExamples(4096, &exs)) for (auto& e : exs) { PS_CHECK(w.WriteProtocolMessage(e)); ++n; }
  return n;
}

}  // namespace PS
