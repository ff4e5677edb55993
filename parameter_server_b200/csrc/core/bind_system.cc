// Python bindings of the host runtime: headers, nodes, the per-node system
// object, customers/apps (overridable from Python) and the shared parameters.
#include "bind_common.h"
#include "ps.h"

namespace PS {

// keeps Python-created apps alive for the life of the process
static std::vector<py::object>& KeepAlive() { static auto* v = new std::vector<py::object>(); return *v; }

// The message handed to a Python handler shares ownership with the executor (which holds it as the
// customer's last request / response), so a handler that defers its answer may keep the object.
static py::object OwnedMessage(Customer* c, Message* m, bool request) {
  std::shared_ptr<Message> held = request ? c->LastRequest() : c->LastResponse();
  if (held && held.get() == m) return py::cast(held);
  return py::cast(m, py::return_value_policy::reference);
}

class PyCustomer : public Customer {
 public:
  using Customer::Customer;
  void ProcessRequest(Message* m) override {
    py::gil_scoped_acquire g;
    py::function f = py::get_override(static_cast<const Customer*>(this), "process_request");
    if (f) f(OwnedMessage(this, m, true));
  }
  void ProcessResponse(Message* m) override {
    py::gil_scoped_acquire g;
    py::function f = py::get_override(static_cast<const Customer*>(this), "process_response");
    if (f) f(OwnedMessage(this, m, false));
  }
};

class PyApp : public App {
 public:
  using App::App;
  void ProcessRequest(Message* m) override {
    py::gil_scoped_acquire g;
    py::function f = py::get_override(static_cast<const App*>(this), "process_request");
    if (f) f(OwnedMessage(this, m, true));
  }
  void ProcessResponse(Message* m) override {
    py::gil_scoped_acquire g;
    py::function f = py::get_override(static_cast<const App*>(this), "process_response");
    if (f) f(OwnedMessage(this, m, false));
  }
  void Run() override {
    py::gil_scoped_acquire g;
    py::function f = py::get_override(static_cast<const App*>(this), "run");
    if (f) { f(); return; }
    py::gil_scoped_release r;
    App::Run();
  }
};

// value arrays travel as raw bytes; expose them typed by the header's value_type
static py::object ValueToNumpy(const Message& m, size_t i) {
  DataType t = i < m.task.value_type.size() ? m.task.value_type[i] : DataType::CHAR;
  const SArray<char>& v = m.value[i];
  switch (t) {
    case DataType::FLOAT: return ToNumpy(SArray<float>(v));
    case DataType::DOUBLE: return ToNumpy(SArray<double>(v));
    case DataType::INT32: return ToNumpy(SArray<int32_t>(v));
    case DataType::INT64: return ToNumpy(SArray<int64_t>(v));
    case DataType::UINT32: return ToNumpy(SArray<uint32_t>(v));
    case DataType::UINT64: return ToNumpy(SArray<uint64_t>(v));
    case DataType::UINT8: return ToNumpy(SArray<uint8_t>(v));
    default: return ToNumpy(SArray<int8_t>(v));
  }
}

struct SumEntry {
  float v = 0;
  void Get(float* d, void*) { *d = v; }
  void Set(const float* d, void*) { v += *d; }
};
struct NoState { void Update() {} };
struct SumUpdater {
  void Init(int, size_t n, float* d) { memset(d, 0, n * sizeof(float)); }
  void Update(int, size_t n, const float* recv, float* d) { for (size_t i = 0; i < n; ++i) d[i] += recv[i]; }
};
typedef KVVector<uint64_t, float> KVVectorF;
typedef KVMap<uint64_t, float, SumEntry, NoState> KVMapSum;
typedef KVLayer<float, SumUpdater> KVLayerSum;

void BindSystem(py::module& m) {
  m.attr("kServerGroup") = kServerGroup;
  m.attr("kWorkerGroup") = kWorkerGroup;
  m.attr("kCompGroup") = kCompGroup;
  m.attr("kReplicaGroup") = kReplicaGroup;
  m.attr("kOwnerGroup") = kOwnerGroup;
  m.attr("kLiveGroup") = kLiveGroup;
  m.attr("kMaxKey") = kMaxKey;
  m.attr("SGD_REQUEST_WORKLOAD") = (int)SGDCall::REQUEST_WORKLOAD;
  m.attr("SGD_UPDATE_MODEL") = (int)SGDCall::UPDATE_MODEL;
  m.attr("SGD_SAVE_MODEL") = (int)SGDCall::SAVE_MODEL;
  m.attr("SGD_ROUND_LIMIT") = (int)SGDCall::ROUND_LIMIT;

  py::class_<Range<Key>>(m, "KeyRange")
      .def(py::init<Key, Key>(), py::arg("begin") = 0, py::arg("end") = kMaxKey)
      .def_static("all", &Range<Key>::All)
      .def_property_readonly("begin", [](const Range<Key>& r) { return r.begin(); })
      .def_property_readonly("end", [](const Range<Key>& r) { return r.end(); })
      .def("size", &Range<Key>::size)
      .def("valid", &Range<Key>::valid)
      .def("empty", &Range<Key>::empty)
      .def("even_divide", &Range<Key>::EvenDivide)
      .def("set_intersection", &Range<Key>::SetIntersection)
      .def("set_union", &Range<Key>::SetUnion)
      .def("contains", [](const Range<Key>& r, Key k) { return r.contains(k); })
      .def("__eq__", &Range<Key>::operator==)
      .def("__repr__", &Range<Key>::ToString);

  py::class_<Node> node(m, "Node");
  py::enum_<Node::Role>(node, "Role")
      .value("SERVER", Node::SERVER).value("WORKER", Node::WORKER).value("SCHEDULER", Node::SCHEDULER)
      .value("GROUP", Node::GROUP).value("UNUSED", Node::UNUSED);
  node.def(py::init<>())
      .def_readwrite("role", &Node::role).def_readwrite("id", &Node::id).def_readwrite("rank", &Node::rank)
      .def_readwrite("hostname", &Node::hostname).def_readwrite("port", &Node::port)
      .def_readwrite("key", &Node::key)
      .def("__repr__", &Node::ShortDebugString);
  m.def("parse_node", &Van::ParseNode);

  py::class_<FilterConfig> fc(m, "FilterConfig");
  py::enum_<FilterConfig::Type>(fc, "Type")
      .value("KEY_CACHING", FilterConfig::KEY_CACHING).value("COMPRESSING", FilterConfig::COMPRESSING)
      .value("FIXING_FLOAT", FilterConfig::FIXING_FLOAT).value("NOISE", FilterConfig::NOISE);
  fc.def(py::init([](FilterConfig::Type t, int num_bytes, bool clear, float mean, float std) {
           FilterConfig c; c.type = t; c.num_bytes = num_bytes; c.clear_cache_if_done = clear; c.mean = mean; c.std = std;
           return c;
         }), py::arg("type"), py::arg("num_bytes") = 3, py::arg("clear_cache_if_done") = false,
         py::arg("mean") = 0.f, py::arg("std") = 1.f)
      .def_readwrite("type", &FilterConfig::type).def_readwrite("num_bytes", &FilterConfig::num_bytes)
      .def_readwrite("clear_cache_if_done", &FilterConfig::clear_cache_if_done)
      .def_readwrite("signature", &FilterConfig::signature)
      .def_readwrite("has_signature", &FilterConfig::has_signature)
      .def_readwrite("uncompressed_size", &FilterConfig::uncompressed_size)
      .def("set_range", [](FilterConfig& c, float lo, float hi) {
        FilterConfig::FixedFloat f; f.has_min = f.has_max = true; f.min_value = lo; f.max_value = hi;
        c.fixed_point.push_back(f);
      });

  py::class_<ParamCall>(m, "ParamCall")
      .def_readwrite("push", &ParamCall::push).def_readwrite("op", &ParamCall::op)
      .def_readwrite("replica", &ParamCall::replica);

  py::class_<Task>(m, "Task")
      .def(py::init<>())
      .def_readwrite("control", &Task::control).def_readwrite("request", &Task::request)
      .def_readwrite("customer_id", &Task::customer_id)
      .def_property("time", [](const Task& t) { return t.time; }, [](Task& t, int v) { t.set_time(v); })
      .def_readwrite("wait_time", &Task::wait_time)
      .def_property("key_range", [](const Task& t) { return t.key_range; },
                    [](Task& t, const Range<Key>& r) { t.set_key_range(r); })
      .def_readwrite("key_channel", &Task::key_channel).def_readwrite("has_key", &Task::has_key)
      .def_readwrite("filter", &Task::filter).def_readwrite("more", &Task::more)
      .def_property("msg", [](const Task& t) { return py::bytes(t.msg); },
                    [](Task& t, const std::string& s) { t.msg = s; })
      .def_readwrite("param", &Task::param).def_readwrite("has_param", &Task::has_param)
      // the SGD call of a task (learner/proto/sgd.proto:5-26): command, workload, round lease
      .def_readonly("has_sgd", &Task::has_sgd)
      .def_property("sgd_cmd", [](const Task& t) { return t.has_sgd ? (int)t.sgd.cmd : 0; },
                    [](Task& t, int c) { t.mutable_sgd()->cmd = (SGDCall::Command)c; })
      .def_property("sgd_load_ids", [](const Task& t) { return t.sgd.load.id; },
                    [](Task& t, const std::vector<int>& ids) { t.mutable_sgd()->load.id = ids; t.sgd.has_load = true; })
      .def_property_readonly("sgd_load_files", [](const Task& t) { return t.sgd.load.data.file; })
      .def_property("sgd_load_finished", [](const Task& t) { return t.sgd.load.finished; },
                    [](Task& t, bool f) { t.mutable_sgd()->load.finished = f; })
      .def_property("sgd_round_limit", [](const Task& t) { return t.sgd.round_limit; },
                    [](Task& t, int64_t v) { t.mutable_sgd()->round_limit = v; })
      .def_property("sgd_final_round", [](const Task& t) { return t.sgd.final_round; },
                    [](Task& t, bool v) { t.mutable_sgd()->final_round = v; })
      .def("serialize", [](const Task& t) { return py::bytes(t.Serialize()); })
      .def_static("parse", [](const std::string& s) { Task t; PS_CHECK(t.Parse(s.data(), s.size())); return t; })
      .def("__repr__", &Task::ShortDebugString);

  py::class_<Message, std::shared_ptr<Message>>(m, "Message")
      .def(py::init<>())
      .def(py::init<const Task&>())
      .def_readwrite("task", &Message::task)
      .def_readwrite("sender", &Message::sender).def_readwrite("recver", &Message::recver)
      .def_readwrite("replied", &Message::replied).def_readwrite("finished", &Message::finished)
      .def_readwrite("valid", &Message::valid)
      .def_property("callback", [](Message& msg) { return msg.callback; },
                    [](Message& msg, py::object f) {
                      if (f.is_none()) { msg.callback = nullptr; return; }
                      auto holder = HoldPython(f);
                      msg.callback = [holder]() { py::gil_scoped_acquire g; (*holder)(); };
                    })
      .def("set_key", [](Message& msg, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> k) {
        msg.set_key(FromNumpy<uint64_t>(k));
      })
      .def("key", [](const Message& msg) { return ToNumpy(SArray<uint64_t>(msg.key)); })
      .def("add_value", [](Message& msg, py::array_t<float, py::array::c_style | py::array::forcecast> v) {
        msg.add_value(FromNumpy<float>(v));
      })
      .def("add_value_f64", [](Message& msg, py::array_t<double, py::array::c_style | py::array::forcecast> v) {
        msg.add_value(FromNumpy<double>(v));
      })
      .def("num_values", [](const Message& msg) { return msg.value.size(); })
      .def("value", [](const Message& msg, size_t i) { PS_CHECK_LT(i, msg.value.size()); return ValueToNumpy(msg, i); })
      .def("value_bytes", [](const Message& msg, size_t i) { return msg.value[i].size(); })
      .def("key_bytes", [](const Message& msg) { return msg.key.size(); })
      .def("mem_size", &Message::mem_size)
      .def("__repr__", &Message::ShortDebugString);

  m.def("slice_message", [](const Message& msg, const std::vector<Range<Key>>& krs) {
    std::vector<std::shared_ptr<Message>> out;
    std::vector<Message*> ptrs;
    for (size_t i = 0; i < krs.size(); ++i) { out.push_back(std::make_shared<Message>(msg.task)); ptrs.push_back(out.back().get()); }
    SliceKOFVMessage<uint64_t>(msg, krs, &ptrs);
    return out;
  });

  py::class_<Options>(m, "Options")
      .def(py::init<>())
      .def_static("parse", [](const std::vector<std::string>& a) { return Options::Parse(a); })
      .def("init_from_env", &Options::InitFromEnv)
      .def_readwrite("num_servers", &Options::num_servers).def_readwrite("num_workers", &Options::num_workers)
      .def_readwrite("num_threads", &Options::num_threads).def_readwrite("num_replicas", &Options::num_replicas)
      .def_readwrite("my_node", &Options::my_node).def_readwrite("scheduler", &Options::scheduler)
      .def_readwrite("interface", &Options::interface)
      .def_readwrite("app_file", &Options::app_file).def_readwrite("app_conf", &Options::app_conf)
      .def_readwrite("key_start", &Options::key_start).def_readwrite("key_end", &Options::key_end)
      .def_readwrite("local", &Options::local).def_readwrite("report_interval", &Options::report_interval)
      .def_readwrite("log_dir", &Options::log_dir)
      .def_readwrite("exit_on_scheduler_loss", &Options::exit_on_scheduler_loss)
      .def_readwrite("rest", &Options::rest);
  m.def("free_port", &Env::FreePort);
  m.def("local_ip", &Env::LocalIP, py::arg("interface") = "");

  py::class_<Postoffice>(m, "Postoffice")
      .def(py::init<>())
      .def_static("instance", &Postoffice::instance, py::return_value_policy::reference)
      .def("run", &Postoffice::Run, py::call_guard<py::gil_scoped_release>())
      .def("start", &Postoffice::Start, py::call_guard<py::gil_scoped_release>())
      .def("stop", &Postoffice::Stop, py::call_guard<py::gil_scoped_release>())
      .def("my_node", [](Postoffice& p) { return p.manager().van().my_node(); })
      .def("scheduler_node", [](Postoffice& p) { return p.manager().van().scheduler(); })
      .def("nodes", [](Postoffice& p) { return p.manager().nodes(); })
      .def("num_workers", [](Postoffice& p) { return p.manager().num_workers(); })
      .def("num_servers", [](Postoffice& p) { return p.manager().num_servers(); })
      .def("next_customer_id", [](Postoffice& p) { return p.manager().NextCustomerID(); })
      .def("wait_servers_ready", [](Postoffice& p) { p.manager().WaitServersReady(); }, py::call_guard<py::gil_scoped_release>())
      .def("wait_workers_ready", [](Postoffice& p) { p.manager().WaitWorkersReady(); }, py::call_guard<py::gil_scoped_release>())
      .def("app", [](Postoffice& p) { return p.manager().app(); }, py::return_value_policy::reference)
      .def("sent_bytes", [](Postoffice& p) { return p.manager().van().sent_bytes(); })
      .def("received_bytes", [](Postoffice& p) { return p.manager().van().received_bytes(); })
      .def("statistic", [](Postoffice& p) { return p.manager().van().Statistic(); })
      .def("add_node_failure_handler", [](Postoffice& p, py::function f) {
        auto holder = HoldPython(f);
        p.manager().AddNodeFailureHandler([holder](const NodeID& id) { py::gil_scoped_acquire g; (*holder)(id); });
      })
      .def("node_disconnected", [](Postoffice& p, const NodeID& id) { p.manager().NodeDisconnected(id); },
           py::call_guard<py::gil_scoped_release>())
      .def("remove_node", [](Postoffice& p, const NodeID& id) { p.manager().RemoveNode(id); },
           py::call_guard<py::gil_scoped_release>());

  auto add_customer_api = [](auto& cls) {
    typedef typename std::remove_reference<decltype(cls)>::type::type C;
    cls.def("submit", [](C& c, const Task& t, const NodeID& recver) { return c.Submit(t, recver); },
            py::call_guard<py::gil_scoped_release>())
        .def("submit_message", [](C& c, Message& msg) { return c.Submit(&msg); }, py::call_guard<py::gil_scoped_release>())
        .def("wait", &C::Wait, py::call_guard<py::gil_scoped_release>())
        .def("last_request", &C::LastRequest).def("last_response", &C::LastResponse)
        .def("wait_received_request", &C::WaitReceivedRequest, py::call_guard<py::gil_scoped_release>())
        .def("finish_received_request", &C::FinishReceivedRequest, py::call_guard<py::gil_scoped_release>())
        .def("num_done_received_request", &C::NumDoneReceivedRequest)
        .def("reply", [](C& c, Message& req, const Task& resp) { c.Reply(&req, resp); },
             py::call_guard<py::gil_scoped_release>())
        .def("reply", [](C& c, Message& req) { c.Reply(&req); }, py::call_guard<py::gil_scoped_release>())
        .def("reply_message", [](C& c, Message& req, Message& resp) { c.Reply(&req, &resp); },
             py::call_guard<py::gil_scoped_release>())
        .def("id", &C::id)
        .def("my_node", [](C& c) { return c.sys().manager().van().my_node(); })
        .def("num_alive", [](C& c, const NodeID& id) { return c.executor()->NumAlive(id); });
  };

  py::class_<Customer, PyCustomer> customer(m, "Customer");
  customer.def(py::init<int, Postoffice*>(), py::arg("id"), py::arg("po") = nullptr, py::keep_alive<1, 3>());
  add_customer_api(customer);

  py::class_<App, Customer, PyApp> app(m, "App");
  app.def(py::init<Postoffice*, int>(), py::arg("po") = nullptr, py::arg("id") = 0, py::keep_alive<1, 2>());
  app.def("run", [](App& a) { a.App::Run(); }, py::call_guard<py::gil_scoped_release>());
  m.def("set_app_factory", [](py::function f) {
    // The factory lives in a C++ static that is destroyed after the interpreter has
    // gone, so it must not own a Python reference: the callable is held by a pointer
    // that is replaced here (with the GIL held) and deliberately never freed at exit.
    static py::object* current = nullptr;
    delete current;
    current = new py::object(f);
    App::external_ownership() = true;
    App::SetFactory([](const std::string& conf, Postoffice* po) -> App* {
      py::gil_scoped_acquire g;
      py::object o = (*current)(conf, py::cast(po, py::return_value_policy::reference));
      KeepAlive().push_back(o);
      return o.cast<App*>();
    });
  });

  // ---- parameters
  py::class_<Parameter, Customer, std::unique_ptr<Parameter, py::nodelete>>(m, "Parameter");
  m.def("request", [](int channel, int ts, const std::vector<int>& wait, py::object filters, py::object key_range) {
    std::vector<FilterConfig> f;
    if (!filters.is_none()) f = filters.cast<std::vector<FilterConfig>>();
    Range<Key> kr = key_range.is_none() ? Range<Key>::All() : key_range.cast<Range<Key>>();
    return Parameter::Request(channel, ts, wait, f, kr);
  }, py::arg("channel"), py::arg("ts") = -1, py::arg("wait") = std::vector<int>(), py::arg("filters") = py::none(),
     py::arg("key_range") = py::none());

  py::class_<KVVectorF, Parameter>(m, "KVVector")
      .def(py::init<bool, int, int, Postoffice*>(), py::arg("buffer_value") = false, py::arg("k") = 1,
           py::arg("id") = -1, py::arg("po") = nullptr, py::keep_alive<1, 5>())
      .def("push", [](KVVectorF& kv, const Task& t, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> keys,
                      std::vector<py::array_t<float, py::array::c_style | py::array::forcecast>> values, py::object cb) {
        SArray<uint64_t> k = FromNumpy<uint64_t>(keys);
        std::vector<SArray<float>> vals;
        for (auto& v : values) vals.push_back(FromNumpy<float>(v));
        std::function<void()> f;
        if (!cb.is_none()) { auto h = HoldPython(cb); f = [h]() { py::gil_scoped_acquire g; (*h)(); }; }
        py::gil_scoped_release r;
        return kv.Push(t, k, vals, f);
      }, py::arg("task"), py::arg("keys"), py::arg("values") = std::vector<py::array_t<float>>(), py::arg("callback") = py::none())
      .def("pull", [](KVVectorF& kv, const Task& t, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> keys, py::object cb) {
        SArray<uint64_t> k = FromNumpy<uint64_t>(keys);
        std::function<void()> f;
        if (!cb.is_none()) { auto h = HoldPython(cb); f = [h]() { py::gil_scoped_acquire g; (*h)(); }; }
        py::gil_scoped_release r;
        return kv.Pull(t, k, f);
      }, py::arg("task"), py::arg("keys"), py::arg("callback") = py::none())
      .def("set_channel", [](KVVectorF& kv, int chl, py::array_t<uint64_t, py::array::c_style | py::array::forcecast> keys,
                             py::array_t<float, py::array::c_style | py::array::forcecast> values) {
        auto& c = kv[chl];
        c.key = FromNumpy<uint64_t>(keys);
        c.value = FromNumpy<float>(values);
      })
      .def("keys", [](KVVectorF& kv, int chl) { return ToNumpy(kv[chl].key); })
      .def("values", [](KVVectorF& kv, int chl) { return ToNumpy(kv[chl].value); })
      .def("clear", &KVVectorF::Clear)
      .def("buffer", [](KVVectorF& kv, int ts) {
        auto& b = kv.buffer(ts);
        py::dict d;
        d["channel"] = b.channel;
        d["idx_range"] = py::make_tuple(b.idx_range.begin(), b.idx_range.end());
        py::list vals;
        for (auto& v : b.values) vals.append(ToNumpy(v));
        d["values"] = vals;
        return d;
      })
      .def("clear_buffer", &KVVectorF::ClearBuffer)
      .def("clear_filter", &KVVectorF::ClearFilter)
      .def("write_to_file", &KVVectorF::WriteToFile);

  py::class_<KVMapSum, Parameter>(m, "KVMapSum")
      .def(py::init<int, int, Postoffice*>(), py::arg("k") = 1, py::arg("id") = -1, py::arg("po") = nullptr,
           py::keep_alive<1, 4>())
      .def("size", &KVMapSum::size)
      .def("write_to_file", &KVMapSum::WriteToFile);

  py::class_<KVLayerSum, Parameter>(m, "KVLayerSum")
      .def(py::init([](size_t thr, int id, Postoffice* po) {
             auto* l = new KVLayerSum(thr, id, po);
             l->set_updater(new SumUpdater());
             return l;
           }), py::arg("partition_thr") = 1000, py::arg("id") = -1, py::arg("po") = nullptr, py::keep_alive<1, 4>())
      .def("push", [](KVLayerSum& l, const Task& t, py::array_t<float, py::array::c_style | py::array::forcecast> data) {
        std::vector<float> copy(data.data(), data.data() + data.size());
        py::gil_scoped_release r;
        return l.Push(t, copy.data(), copy.size(), false);
      })
      .def("pull", [](KVLayerSum& l, const Task& t, py::array_t<float, py::array::c_style> out, py::object cb) {
        std::function<void()> f;
        if (!cb.is_none()) { auto h = HoldPython(cb); f = [h]() { py::gil_scoped_acquire g; (*h)(); }; }
        float* p = out.mutable_data();
        size_t n = out.size();
        py::gil_scoped_release r;
        return l.Pull(t, p, n, f);
      }, py::arg("task"), py::arg("out"), py::arg("callback") = py::none())
      .def("layer", [](KVLayerSum& l, int id) { return ToNumpy(l.layer(id)); });
}

}  // namespace PS
