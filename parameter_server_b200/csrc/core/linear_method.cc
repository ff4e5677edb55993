#include "linear_method.h"

namespace PS {
namespace LM {

// Loads every model_input file ("key value" per line), streams validation_data
// in chunks, scores by hash lookup and prints AUC / accuracy / logloss.
void ModelEvaluation::Run() {
  if (!sys_->manager().IsScheduler()) return;
  std::unordered_map<Key, Real> weight;
  DataConfig model = searchFiles(conf_.model_input);
  PS_NOTICE("find %d model files", (int)model.file.size());
  for (auto& f : model.file) {
    std::ifstream in(f);
    Key k;
    Real v;
    while (in >> k >> v) weight[k] = v;
  }
  num_weights = weight.size();
  PS_NOTICE("load %lu model entries", (unsigned long)num_weights);
  DataConfig data = conf_.validation_data;
  data.ignore_feature_group = true;
  StreamReader<Real> reader(data);
  SArray<Real> label, margin;
  SArray<Real> y;
  std::vector<std::shared_ptr<SparseMatrix<uint64_t, Real>>> mats;
  while (reader.readMatrices(100000, &y, &mats)) {
    size_t n = y.size();
    SArray<Real> xw(n);
    xw.SetZero();
    for (auto& m : mats) {
      for (size_t i = 0; i < n; ++i) {
        Real s = 0;
        for (size_t j = m->offset()[i]; j < m->offset()[i + 1]; ++j) {
          auto it = weight.find(m->index()[j]);
          if (it != weight.end()) s += it->second * (m->binary() ? 1 : m->value()[j]);
        }
        xw[i] += s;
      }
    }
    label.append(y);
    margin.append(xw);
  }
  num_examples = label.size();
  PS_NOTICE("load %lu examples", (unsigned long)num_examples);
  if (num_examples == 0) return;
  auc = Evaluation<Real>::auc(label, margin);
  accuracy = Evaluation<Real>::accuracy(label, margin);
  logloss = Evaluation<Real>::logloss(label, margin);
  PS_NOTICE("auc: %f", auc);
  PS_NOTICE("accuracy: %f", accuracy);
  PS_NOTICE("logloss: %f", logloss);
}

App* CreateLinearMethod(const std::string& conf_text, Postoffice* po) {
  Config conf = ParseConfig(conf_text);
  if (po == nullptr) po = &Postoffice::instance();
  Node::Role role = po->manager().van().my_node().role;
  if (conf.has_darlin) return CreateDarlin(conf, po);
  if (conf.has_async_sgd) {
    if (role == Node::SCHEDULER) return new AsyncSGDScheduler(conf, po);
    if (role == Node::WORKER) return new AsyncSGDWorker<Real>(conf, po);
    if (role == Node::SERVER) return new AsyncSGDServer<Real>(conf, po);
  }
  if (conf.has_validation_data) return new ModelEvaluation(conf, po);
  PS_CHECK(false) << "the configuration selects no application (async_sgd, darlin or validation_data)";
  return nullptr;
}

}  // namespace LM
}  // namespace PS
