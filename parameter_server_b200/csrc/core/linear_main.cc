// `psb_linear`: the linear-method binary (the reference's build/linear,
// app/linear_method/main.cc:43-46). Every node of the system runs this program:
//   psb_linear -my_node "role:WORKER,hostname:'127.0.0.1',port:9500,id:'W0'" \
//              -scheduler "role:SCHEDULER,..." -num_servers 2 -num_workers 2 -app_file x.conf
#include "linear_method.h"
#include "ps.h"

int main(int argc, char* argv[]) {
  try {
    PS::App::SetFactory([](const std::string& conf, PS::Postoffice* po) { return PS::LM::CreateLinearMethod(conf, po); });
    return PS::RunSystem(argc, argv);
  } catch (const std::exception& e) {
    fprintf(stderr, "psb_linear: %s\n", e.what());
    return 1;
  }
}
