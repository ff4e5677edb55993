#include "customer.h"

#include "postoffice.h"

namespace PS {

Customer::Customer(int id, Postoffice* po)
    : sys_(po ? po : &Postoffice::instance()), id_(id), exec_(*this, sys_) {
  sys_->manager().AddCustomer(this);
  exec_.Start();
}

Customer::~Customer() {
  exec_.Stop();
  sys_->manager().RemoveCustomer(id_);
}

void App::Run() {
  // by default: every server and worker has joined
  sys_->manager().WaitServersReady();
  sys_->manager().WaitWorkersReady();
}

}  // namespace PS
