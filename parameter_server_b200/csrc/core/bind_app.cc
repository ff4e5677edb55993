// Python bindings of the data layer, the learner helpers and the CPU
// linear-method applications.
#include "bind_common.h"
#include "linear_method.h"

namespace PS {

static py::dict TextNodeToDict(const TextNode& n) {
  py::dict d;
  for (auto& s : n.scalars) {
    if (d.contains(s.first.c_str())) {
      py::object cur = d[s.first.c_str()];
      if (py::isinstance<py::list>(cur)) cur.cast<py::list>().append(s.second);
      else { py::list l; l.append(cur); l.append(s.second); d[s.first.c_str()] = l; }
    } else d[s.first.c_str()] = s.second;
  }
  for (auto& c : n.children) {
    py::dict sub = TextNodeToDict(c.second);
    if (d.contains(c.first.c_str())) {
      py::object cur = d[c.first.c_str()];
      if (py::isinstance<py::list>(cur)) cur.cast<py::list>().append(sub);
      else { py::list l; l.append(cur); l.append(sub); d[c.first.c_str()] = l; }
    } else d[c.first.c_str()] = sub;
  }
  return d;
}

static py::dict ExampleToDict(const Example& ex) {
  py::dict d;
  for (auto& s : ex.slot) {
    py::dict sd;
    sd["key"] = py::array_t<uint64_t>(s.key.size(), s.key.data());
    sd["val"] = py::array_t<float>(s.val.size(), s.val.data());
    d[py::int_(s.id)] = sd;
  }
  return d;
}

static DataConfig MakeData(const std::vector<std::string>& files, const std::string& format, const std::string& text,
                           bool ignore_group, int max_lines) {
  TextNode n;
  n.scalars.emplace_back("format", format);
  n.scalars.emplace_back("text", text);
  for (auto& f : files) n.scalars.emplace_back("file", f);
  DataConfig d = LM::ParseData(n);
  d.ignore_feature_group = ignore_group;
  d.max_num_lines_per_file = max_lines;
  return d;
}

void BindApp(py::module& m) {
  m.def("parse_text_proto", [](const std::string& text) { return TextNodeToDict(TextProtoParser::Parse(text)); },
        "protobuf text format -> nested dict (repeated fields become lists)");
  m.def("use_linear_method_factory", []() {
    App::external_ownership() = false;
    App::SetFactory([](const std::string& conf, Postoffice* po) { return LM::CreateLinearMethod(conf, po); });
  }, "every node created afterwards runs the C++ linear-method application selected by its configuration");

  m.def("parse_example", [](const std::string& line, const std::string& text_format, bool ignore_group) {
    TextNode n;
    n.scalars.emplace_back("text", text_format);
    DataConfig d = LM::ParseData(n);
    ExampleParser p;
    p.Init(d.text, ignore_group);
    std::vector<char> buf(line.begin(), line.end());
    buf.push_back('\0');
    Example ex;
    if (!p.ToProto(buf.data(), &ex)) return py::object(py::none());
    return py::object(ExampleToDict(ex));
  }, py::arg("line"), py::arg("text_format"), py::arg("ignore_feature_group") = false);

  typedef StreamReader<float> SR;
  py::class_<SR>(m, "StreamReader")
      .def(py::init([](const std::vector<std::string>& files, const std::string& format, const std::string& text,
                       bool ignore_group, int max_lines) {
             return new SR(MakeData(files, format, text, ignore_group, max_lines));
           }), py::arg("files"), py::arg("format") = "TEXT", py::arg("text") = "LIBSVM",
           py::arg("ignore_feature_group") = false, py::arg("max_num_lines_per_file") = -1)
      .def("set_hash_kernel", &SR::set_hash_kernel)
      .def("set_parse_threads", &SR::set_parse_threads)
      .def("read_matrices", [](SR& r, uint32_t n) -> py::object {
        SArray<float> y;
        std::vector<std::shared_ptr<SparseMatrix<uint64_t, float>>> mats;
        bool ok;
        { py::gil_scoped_release rel; ok = r.readMatrices(n, &y, &mats); }   // parsing needs no interpreter
        if (!ok) return py::none();
        py::list out;
        for (auto& mt : mats) {
          py::dict d;
          d["id"] = mt->info().id;
          d["offset"] = ToNumpy(SArray<uint64_t>(mt->offset()));
          d["index"] = ToNumpy(mt->index());
          d["value"] = ToNumpy(mt->value());
          d["binary"] = mt->binary();
          out.append(d);
        }
        return py::make_tuple(ToNumpy(y), out);
      }, "(labels, [per-slot CSR dict]) of the next n examples, or None at the end");

  py::class_<SlotReader>(m, "SlotReader")
      .def(py::init([](const std::vector<std::string>& files, const std::string& text, const std::string& cache) {
             return new SlotReader(MakeData(files, "TEXT", text, false, -1), cache);
           }), py::arg("files"), py::arg("text") = "LIBSVM", py::arg("cache_dir") = "")
      .def("read", [](SlotReader& r, int threads) {
        ExampleInfo info;
        { py::gil_scoped_release rel; r.Read(&info, threads); }
        py::dict d;
        d["num_ex"] = info.num_ex;
        py::list slots;
        for (auto& s : info.slot) {
          py::dict sd;
          sd["id"] = s.id; sd["nnz_ele"] = s.nnz_ele; sd["nnz_ex"] = s.nnz_ex; sd["min_key"] = s.min_key; sd["max_key"] = s.max_key;
          sd["format"] = (int)s.format;
          slots.append(sd);
        }
        d["slot"] = slots;
        return d;
      }, py::arg("num_threads") = 2)
      .def("index", [](SlotReader& r, int id) { return ToNumpy(r.index(id)); })
      .def("offset", [](SlotReader& r, int id) { return ToNumpy(SArray<uint64_t>(r.offset(id))); })
      .def("value", [](SlotReader& r, int id) { return ToNumpy(r.value(id)); })
      .def("hit_cache", &SlotReader::hit_cache);

  m.def("text_to_records", [](const std::vector<std::string>& files, const std::string& text, const std::string& out) {
    return textToRecords(MakeData(files, "TEXT", text, false, -1), out);
  });
  m.def("search_files", [](const std::vector<std::string>& patterns, py::object hdfs, const std::string& format) {
    DataConfig d; d.file = patterns;
    if (format == "BIN") d.format = DataConfig::BIN;
    if (!hdfs.is_none()) {
      py::dict h = hdfs.cast<py::dict>();
      auto get = [&](const char* k) { return h.contains(k) ? py::str(h[k]).cast<std::string>() : std::string(); };
      d.has_hdfs = true; d.hdfs.home = get("home"); d.hdfs.ugi = get("ugi"); d.hdfs.namenode = get("namenode");
    }
    return searchFiles(d).file;
  }, py::arg("patterns"), py::arg("hdfs") = py::none(), py::arg("format") = "TEXT",
     "files matching the patterns (regular expression in the file part); with hdfs={home, ugi, namenode} the "
     "patterns name HDFS files, the names returned start with hdfs:// and every reader of this process opens "
     "such names through `hadoop fs -cat`");
  m.def("hadoop_fs", []() { return currentHadoopFS(); }, "the command prefix used for hdfs:// files");
  m.def("set_reader_flags", [](uint64_t hash_kernel, bool shuffle_fea_id, int line_limit, int parse_threads) {
    ReaderFlags& f = ReaderFlags::get();
    f.hash_kernel = hash_kernel; f.shuffle_fea_id = shuffle_fea_id; f.line_limit = line_limit;
    if (parse_threads > 0) f.parse_threads = parse_threads;
  }, py::arg("hash_kernel") = 0, py::arg("shuffle_fea_id") = false, py::arg("line_limit") = 0, py::arg("parse_threads") = 0,
     "process-wide defaults of the readers made afterwards: the node flags -hash_kernel, -shuffle_fea_id, -line_limit, -num_threads (0 keeps the current number)");

  m.def("localize", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> offset,
                       py::array_t<uint64_t, py::array::c_style | py::array::forcecast> index, int threads) {
    MatrixInfo info;
    info.type = MatrixInfo::SPARSE_BINARY;
    info.row = SizeR(0, offset.size() - 1);
    info.nnz = index.size();
    SArray<size_t> off(offset.size());
    for (py::ssize_t i = 0; i < offset.size(); ++i) off[i] = offset.data()[i];
    SparseMatrix<uint64_t, float> mat(info, off, FromNumpy<uint64_t>(index), SArray<float>());
    Localizer<uint64_t, float> loc;
    SArray<uint64_t> uniq;
    SArray<uint32_t> cnt;
    loc.CountUniqIndex<uint32_t>(mat, &uniq, &cnt, threads);
    auto X = loc.RemapIndex(uniq);
    return py::make_tuple(ToNumpy(uniq), ToNumpy(cnt), ToNumpy(X->index()));
  }, py::arg("offset"), py::arg("index"), py::arg("threads") = 2,
     "(unique sorted keys, counts, remapped column ids) of a CSR matrix with uint64 columns");

  m.def("spmv", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> offset,
                   py::array_t<uint32_t, py::array::c_style | py::array::forcecast> index, py::object value,
                   py::array_t<float, py::array::c_style | py::array::forcecast> x, size_t cols, bool trans, int threads) {
    MatrixInfo info;
    info.row = SizeR(0, offset.size() - 1);
    info.col = SizeR(0, cols);
    info.nnz = index.size();
    SArray<size_t> off(offset.size());
    for (py::ssize_t i = 0; i < offset.size(); ++i) off[i] = offset.data()[i];
    SArray<float> val;
    if (!value.is_none()) val = FromNumpy<float>(value.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>());
    info.type = val.empty() ? MatrixInfo::SPARSE_BINARY : MatrixInfo::SPARSE;
    SparseMatrix<uint32_t, float> mat(info, off, FromNumpy<uint32_t>(index), val);
    SArray<float> xv = FromNumpy<float>(x);
    SArray<float> y = trans ? mat.transTimes(xv, threads) : mat.times(xv, threads);
    return ToNumpy(y);
  }, py::arg("offset"), py::arg("index"), py::arg("value"), py::arg("x"), py::arg("cols"), py::arg("trans") = false,
     py::arg("threads") = 2);
  m.def("sparse_debug_string", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> offset,
                                  py::array_t<uint32_t, py::array::c_style | py::array::forcecast> index, py::object value,
                                  size_t cols) {
    MatrixInfo info;
    info.row = SizeR(0, offset.size() - 1);
    info.col = SizeR(0, cols);
    info.nnz = index.size();
    SArray<size_t> off(offset.size());
    for (py::ssize_t i = 0; i < offset.size(); ++i) off[i] = offset.data()[i];
    SArray<float> val;
    if (!value.is_none()) val = FromNumpy<float>(value.cast<py::array_t<float, py::array::c_style | py::array::forcecast>>());
    info.type = val.empty() ? MatrixInfo::SPARSE_BINARY : MatrixInfo::SPARSE;
    return SparseMatrix<uint32_t, float>(info, off, FromNumpy<uint32_t>(index), val).debugString();
  }, py::arg("offset"), py::arg("index"), py::arg("value"), py::arg("cols"), "header and first entries of a CSR matrix");

  m.def("transpose_csr", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> offset,
                            py::array_t<uint32_t, py::array::c_style | py::array::forcecast> index, size_t cols) {
    MatrixInfo info;
    info.type = MatrixInfo::SPARSE_BINARY;
    info.row = SizeR(0, offset.size() - 1);
    info.col = SizeR(0, cols);
    info.nnz = index.size();
    SArray<size_t> off(offset.size());
    for (py::ssize_t i = 0; i < offset.size(); ++i) off[i] = offset.data()[i];
    SparseMatrix<uint32_t, float> mat(info, off, FromNumpy<uint32_t>(index), SArray<float>());
    auto t = mat.alterStorage();
    return py::make_tuple(ToNumpy(SArray<uint64_t>(t->offset())), ToNumpy(t->index()));
  });

  m.def("evaluate", [](py::array_t<float, py::array::c_style | py::array::forcecast> label,
                       py::array_t<float, py::array::c_style | py::array::forcecast> predict) {
    SArray<float> y = FromNumpy<float>(label), p = FromNumpy<float>(predict);
    py::dict d;
    d["auc"] = Evaluation<float>::auc(y, p);
    d["accuracy"] = Evaluation<float>::accuracy(y, p);
    d["logloss"] = Evaluation<float>::logloss(y, p);
    AUC h;
    AUC::Data data;
    h.compute(y, p, &data);
    h.merge(data);
    d["auc_histogram"] = h.evaluate();
    return d;
  });

  py::class_<WorkloadPool>(m, "WorkloadPool")
      .def(py::init([](const std::vector<std::string>& files, int replica, bool shuffle) {
             Workload w; w.data.file = files; w.replica = replica; w.shuffle = shuffle;
             return new WorkloadPool(w);
           }), py::arg("files"), py::arg("replica") = 1, py::arg("shuffle") = false)
      .def("assign", [](WorkloadPool& p, const NodeID& node) -> py::object {
        Workload w;
        if (!p.assign(node, &w)) return py::none();
        return py::make_tuple(w.id[0], w.data.file[0]);
      })
      .def("restore", &WorkloadPool::restore).def("finish", &WorkloadPool::finish)
      .def("size", &WorkloadPool::size).def("num_finished", &WorkloadPool::num_finished)
      .def("wait_until_done", &WorkloadPool::waitUtilDone, py::call_guard<py::gil_scoped_release>());

  // scheduler of lock-step device workers (files handed out one at a time, rounds granted in leases)
  py::class_<LockstepSGDScheduler, App>(m, "LockstepSGDScheduler")
      .def(py::init([](const std::vector<std::string>& files, const std::string& format, const std::string& text,
                       int replica, bool shuffle, int lease, Postoffice* po) {
             Workload w;
             w.data = MakeData(files, format, text, true, -1);
             w.replica = replica;
             w.shuffle = shuffle;
             return new LockstepSGDScheduler(w, lease, po);
           }), py::arg("files"), py::arg("format") = "TEXT", py::arg("text") = "LIBSVM", py::arg("replica") = 1,
           py::arg("shuffle") = true, py::arg("lease") = 64, py::arg("po") = nullptr, py::keep_alive<1, 8>())
      .def("round_limit", &LockstepSGDScheduler::round_limit)
      .def("num_workloads", [](LockstepSGDScheduler& s) { return s.pool().size(); })
      .def("num_finished", [](LockstepSGDScheduler& s) { return s.pool().num_finished(); })
      .def("num_examples_processed", &LockstepSGDScheduler::num_examples_processed);

  // progress reports of a worker or server node to the scheduler's monitor (system/monitor.h:60-97,
  // learner/sgd.cc:51-86)
  typedef MonitorSlaver<SGDProgress> Reporter;
  py::class_<Reporter, Customer>(m, "SGDReporter")
      .def(py::init([](Postoffice* po) {
             return new Reporter(po->manager().van().scheduler().id, kMonitorCustomerID, po);
           }), py::arg("po"), py::keep_alive<1, 2>())
      .def("report", [](Reporter& r, std::vector<double> objective, std::vector<double> accuracy, std::vector<double> auc,
                        uint64_t num_examples, uint64_t nnz, double weight_sum, double delta_sum, uint64_t round) {
        SGDProgress p;
        p.objective = objective; p.accuracy = accuracy; p.auc = auc;
        p.num_examples_processed = num_examples; p.nnz = nnz; p.weight_sum = weight_sum; p.delta_sum = delta_sum;
        p.round = round;
        r.Report(p);
      }, py::arg("objective") = std::vector<double>(), py::arg("accuracy") = std::vector<double>(),
         py::arg("auc") = std::vector<double>(), py::arg("num_examples") = 0, py::arg("nnz") = 0,
         py::arg("weight_sum") = 0.0, py::arg("delta_sum") = 0.0, py::arg("round") = 0,
         py::call_guard<py::gil_scoped_release>());

  py::class_<Dashboard>(m, "Dashboard")
      .def(py::init<>())
      .def("add_task", &Dashboard::addTask)
      .def("add_report", [](Dashboard& d, const NodeID& n, py::bytes b) { d.addReport(n, b); })
      .def("title", &Dashboard::title).def("report", &Dashboard::report);
  py::class_<HeartbeatInfo>(m, "HeartbeatInfo")
      .def(py::init<>())
      .def("init", &HeartbeatInfo::init)
      .def("increase_in_bytes", &HeartbeatInfo::increaseInBytes).def("increase_out_bytes", &HeartbeatInfo::increaseOutBytes)
      .def("get", [](HeartbeatInfo& h) { return py::bytes(h.get().Serialize()); });
  py::class_<TaskTracker>(m, "TaskTracker")
      .def(py::init<>())
      .def("start", &TaskTracker::start).def("finish", &TaskTracker::finish)
      .def("wait", &TaskTracker::wait, py::call_guard<py::gil_scoped_release>())
      .def("has_finished", &TaskTracker::hasFinished).def("was_started", &TaskTracker::wasStarted);
}

}  // namespace PS
