// Python bindings of utilities: hashes, sketches, filters (stand-alone
// encode/decode), ordered match.
#include "bind_common.h"
#include "data.h"
#include "evaluation.h"
#include "filter.h"
#include "ordered_match.h"
#include "remote_node.h"

namespace PS {

void BindUtil(py::module& m) {
  m.def("crc32c", [](py::bytes b) { std::string s = b; return crc32c::Value(s.data(), s.size()); });
  m.def("crc32c_extend", [](uint32_t init, py::bytes b) { std::string s = b; return crc32c::Extend(init, s.data(), s.size()); });
  m.def("crc32c_mask", &crc32c::Mask);
  m.def("crc32c_unmask", &crc32c::Unmask);
  m.def("murmurhash3_x86_32", [](py::bytes b, uint32_t seed) {
    std::string s = b; uint32_t out; MurmurHash3_x86_32(s.data(), (int)s.size(), seed, &out); return out;
  });
  m.def("murmurhash3_x86_128", [](py::bytes b, uint32_t seed) {
    std::string s = b; uint32_t out[4]; MurmurHash3_x86_128(s.data(), (int)s.size(), seed, out);
    return py::make_tuple(out[0], out[1], out[2], out[3]);
  });
  m.def("murmurhash3_x64_128", [](py::bytes b, uint32_t seed) {
    std::string s = b; uint64_t out[2]; MurmurHash3_x64_128(s.data(), (int)s.size(), seed, out);
    return py::make_tuple(out[0], out[1]);
  });
  m.def("sketch_hash", [](uint64_t k) { return Sketch::hash(k); });
  m.def("res_usage", []() {
    py::dict d;
    d["my_phy_mem_mb"] = ResUsage::myPhyMem(); d["my_vir_mem_mb"] = ResUsage::myVirMem();
    d["host_total_mem_mb"] = ResUsage::hostTotalMem(); d["host_in_use_mem_mb"] = ResUsage::hostInUseMem();
    return d;
  }, "memory of this process and of the machine, in MB");
  m.def("hwtic", []() { return hwtic(); }, "time-stamp counter now");
  m.def("hwtoc", [](uint64_t start) { return hwtoc(start); }, "cycles since hwtic()");
  m.def("read_file", [](const std::string& name) -> py::object {
    std::string out;
    bool ok;
    { py::gil_scoped_release r; ok = readFileToString(name, &out); }
    if (!ok) return py::none();
    return py::bytes(out);
  }, "whole contents of a plain, .gz or s3:// file (None if it cannot be opened)");
  m.def("s3_file_url", &s3FileUrl);
  m.def("s3_directory_url", &s3DirectoryUrl);

  typedef CountMin<uint64_t, uint8_t> CM8;
  py::class_<CM8>(m, "CountMin")
      .def(py::init<>())
      .def("resize", [](CM8& c, int n, int k, int vmax) { c.resize(n, k, (uint8_t)vmax); })
      .def("insert", [](CM8& c, uint64_t key, int cnt) { c.insert(key, (uint8_t)cnt); })
      .def("query", [](const CM8& c, uint64_t key) { return (int)c.query(key); })
      .def("insert_many", [](CM8& c, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> k,
                             py::array_t<uint8_t, py::array::c_style | py::array::forcecast> v) {
        for (py::ssize_t i = 0; i < k.size(); ++i) c.insert(k.data()[i], v.data()[i]);
      })
      .def("query_many", [](const CM8& c, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> k) {
        py::array_t<uint8_t> out(k.size());
        for (py::ssize_t i = 0; i < k.size(); ++i) out.mutable_data()[i] = c.query(k.data()[i]);
        return out;
      })
      .def("data", [](const CM8& c) { return ToNumpy(c.data()); });
  typedef BloomFilter<uint64_t> BF;
  py::class_<BF>(m, "BloomFilter").def(py::init<int, int>()).def("insert", &BF::insert).def("query", &BF::query);
  typedef BlockBloomFilter<uint64_t> BBF;
  py::class_<BBF>(m, "BlockBloomFilter").def(py::init<size_t, int>()).def("insert", &BBF::insert).def("query", &BBF::query);
  py::class_<Bitmap>(m, "Bitmap")
      .def(py::init<uint32_t, bool>(), py::arg("size"), py::arg("value") = false)
      .def("set", &Bitmap::set).def("clear", (void (Bitmap::*)(uint32_t)) & Bitmap::clear)
      .def("test", &Bitmap::test).def("fill", &Bitmap::fill).def("nnz", &Bitmap::nnz).def("size", &Bitmap::size);

  typedef FreqencyFilter<uint64_t, uint8_t> FF;
  py::class_<FF>(m, "FreqencyFilter")
      .def(py::init<>())
      .def("resize", &FF::Resize)
      .def("insert_keys", [](FF& f, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> k,
                             py::array_t<uint8_t, py::array::c_style | py::array::forcecast> c) {
        f.InsertKeys(FromNumpy<uint64_t>(k), FromNumpy<uint8_t>(c));
      })
      .def("query_keys", [](const FF& f, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> k, int thr) {
        return ToNumpy(f.QueryKeys(FromNumpy<uint64_t>(k), thr));
      });

  // a peer's filter chain, for stand-alone encode/decode
  py::class_<RemoteNode>(m, "FilterChain")
      .def(py::init<>())
      .def("encode", [](RemoteNode& r, Message& msg) { r.EncodeMessage(&msg); })
      .def("decode", [](RemoteNode& r, Message& msg) { r.DecodeMessage(&msg); })
      .def("set_fixing_float_seed", [](RemoteNode& r, unsigned seed) {
        FilterConfig c; c.type = FilterConfig::FIXING_FLOAT;
        static_cast<FixingFloatFilter*>(r.FilterFor(c))->set_seed(seed);
      });
  m.def("sparse_filter_mark", []() { SparseFilter f; float v = 0; f.mark(&v); return v; });

  m.def("ordered_match", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> src_key,
                            py::array_t<float, py::array::c_style | py::array::forcecast> src_val,
                            py::array_t<uint64_t, py::array::c_style | py::array::forcecast> dst_key,
                            py::array_t<float, py::array::c_style | py::array::forcecast> dst_val, int k, int op, int threads) {
    SArray<float> dv = FromNumpy<float>(dst_val);
    size_t n = ParallelOrderedMatch(FromNumpy<uint64_t>(src_key), FromNumpy<float>(src_val), FromNumpy<uint64_t>(dst_key),
                                    &dv, k, (AssignOp)op, threads);
    return py::make_tuple(n, ToNumpy(dv));
  }, py::arg("src_key"), py::arg("src_val"), py::arg("dst_key"), py::arg("dst_val"), py::arg("k") = 1,
     py::arg("op") = 0, py::arg("threads") = 2);
  m.def("parallel_sort_u64", [](py::array_t<uint64_t, py::array::c_style | py::array::forcecast> a, int threads) {
    SArray<uint64_t> s = FromNumpy<uint64_t>(a);
    ParallelSort(&s, threads, [](uint64_t x, uint64_t y) { return x < y; });
    return ToNumpy(s);
  });
}

}  // namespace PS
