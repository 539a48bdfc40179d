// InfiniBand verbs layer (see ib.hpp). The verbs library is loaded with dlopen; every call goes through IbvApi.
#include "ib.hpp"

#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <mutex>
#include <sstream>

#include <cuda_runtime.h>

#include <mscclpp/env.hpp>
#include <mscclpp/errors.hpp>

#include "cuda_driver.hpp"
#include "logger.hpp"

namespace mscclpp {

// ------------------------------------------------------------------------------------------ IbvApi
namespace {
std::mutex g_apiMutex;
std::shared_ptr<const IbvApi> g_api;
std::string g_apiError;
}  // namespace

struct IbvApiLoader {
  static std::shared_ptr<const IbvApi> load(std::string& error) {
    auto api = std::make_shared<IbvApi>();
    std::vector<std::string> candidates;
    if (!env()->ibvSo.empty()) candidates.push_back(env()->ibvSo);
    else candidates = {"libibverbs.so.1", "libibverbs.so"};
    for (const auto& c : candidates) {
      api->handle_ = ::dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (api->handle_ != nullptr) {
        api->path = c;
        break;
      }
      error = std::string("cannot load ") + c + ": " + ::dlerror();
    }
    if (api->handle_ == nullptr) return nullptr;
    bool ok = true;
    auto need = [&](auto& slot, const char* name, bool required = true) {
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(::dlsym(api->handle_, name));
      if (slot == nullptr && required) {
        error = api->path + " has no symbol " + name;
        ok = false;
      }
    };
    need(api->getDeviceList, "ibv_get_device_list");
    need(api->freeDeviceList, "ibv_free_device_list");
    need(api->getDeviceName, "ibv_get_device_name");
    need(api->openDevice, "ibv_open_device");
    need(api->closeDevice, "ibv_close_device");
    need(api->queryDevice, "ibv_query_device");
    need(api->queryPort, "ibv_query_port");
    need(api->queryGid, "ibv_query_gid");
    need(api->allocPd, "ibv_alloc_pd");
    need(api->deallocPd, "ibv_dealloc_pd");
    need(api->regMr, "ibv_reg_mr");
    need(api->regDmabufMr, "ibv_reg_dmabuf_mr", false);
    need(api->deregMr, "ibv_dereg_mr");
    need(api->createCq, "ibv_create_cq");
    need(api->destroyCq, "ibv_destroy_cq");
    need(api->createQp, "ibv_create_qp");
    need(api->modifyQp, "ibv_modify_qp");
    need(api->destroyQp, "ibv_destroy_qp");
    need(api->wcStatusStr, "ibv_wc_status_str", false);
    need(api->postSendSym_, "ibv_post_send", false);
    need(api->postRecvSym_, "ibv_post_recv", false);
    need(api->pollCqSym_, "ibv_poll_cq", false);
    if (!ok) {
      ::dlclose(api->handle_);
      return nullptr;
    }
    return api;
  }
};

std::shared_ptr<const IbvApi> IbvApi::get() {
  std::lock_guard<std::mutex> lock(g_apiMutex);
  if (!g_api) {
    g_api = IbvApiLoader::load(g_apiError);
    if (!g_api) throw Error("InfiniBand is not available: " + g_apiError, ErrorCode::SystemError);
  }
  return g_api;
}

bool IbvApi::available() {
  try {
    return get() != nullptr;
  } catch (const Error&) {
    return false;
  }
}

int IbvApi::postSend(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) const {
  return postSendSym_ != nullptr ? postSendSym_(qp, wr, bad) : qp->context->ops.post_send(qp, wr, bad);
}
int IbvApi::postRecv(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad) const {
  return postRecvSym_ != nullptr ? postRecvSym_(qp, wr, bad) : qp->context->ops.post_recv(qp, wr, bad);
}
int IbvApi::pollCq(ibv_cq* cq, int n, ibv_wc* wc) const {
  return pollCqSym_ != nullptr ? pollCqSym_(cq, n, wc) : cq->context->ops.poll_cq(cq, n, wc);
}

std::vector<std::string> ibDeviceNamesFromLibrary() {
  std::vector<std::string> names;
  if (!IbvApi::available()) return names;
  auto api = IbvApi::get();
  int n = 0;
  ibv_device** list = api->getDeviceList(&n);
  if (list == nullptr) return names;
  for (int i = 0; i < n; i++) names.emplace_back(api->getDeviceName(list[i]));
  api->freeDeviceList(list);
  std::sort(names.begin(), names.end());
  const std::string forced = env()->hcaDevices;
  if (!forced.empty()) {
    std::vector<std::string> picked;
    std::stringstream ss(forced);
    std::string item;
    while (std::getline(ss, item, ',')) {
      if (!item.empty() && std::find(names.begin(), names.end(), item) != names.end()) picked.push_back(item);
    }
    return picked;
  }
  return names;
}

// ------------------------------------------------------------------------------------------ IbMr
namespace {
constexpr int kMrAccess = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ | IBV_ACCESS_REMOTE_ATOMIC;

bool isDevicePointer(const void* p) {
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}
}  // namespace

IbMr::IbMr(std::shared_ptr<const IbvApi> api, ibv_pd* pd, void* buff, size_t size) : api_(std::move(api)), buff_(buff), size_(size) {
  if (size == 0) throw Error("cannot register an empty memory region", ErrorCode::InvalidUsage);
  // Device memory: prefer a DMA-BUF export of the page-aligned range (works without the peer-memory kernel module);
  // fall back to plain registration, which needs that module for device addresses.
  const CudaDriver* drv = CudaDriver::tryGet();
  if (api_->regDmabufMr != nullptr && drv != nullptr && drv->cuMemGetHandleForAddressRange != nullptr && isDevicePointer(buff)) {
    const long page = ::sysconf(_SC_PAGESIZE);
    const uint64_t addr = reinterpret_cast<uint64_t>(buff);
    const uint64_t begin = addr / page * page;
    const uint64_t end = (addr + size + page - 1) / page * page;
    int fd = -1;
    if (drv->cuMemGetHandleForAddressRange(&fd, begin, end - begin, CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0) == CUDA_SUCCESS && fd >= 0) {
      mr_ = api_->regDmabufMr(pd, addr - begin, size, addr, fd, kMrAccess);
      ::close(fd);
      dmabuf_ = mr_ != nullptr;
    }
  }
  if (mr_ == nullptr) mr_ = api_->regMr(pd, buff, size, kMrAccess);
  if (mr_ == nullptr) {
    std::ostringstream os;
    os << "ibv_reg_mr failed for " << size << " bytes at " << buff;
    throw IbError(os.str(), errno);
  }
}

IbMr::~IbMr() {
  if (mr_ != nullptr) (void)api_->deregMr(mr_);
}

IbMrInfo IbMr::info() const {
  IbMrInfo i;
  i.addr = reinterpret_cast<uint64_t>(buff_);
  i.rkey = mr_->rkey;
  return i;
}
uint32_t IbMr::lkey() const { return mr_->lkey; }

// ------------------------------------------------------------------------------------------ IbQp
IbQp::IbQp(std::shared_ptr<const IbvApi> api, ibv_context* ctx, ibv_pd* pd, int port, int gidIndex, const Limits& limits)
    : api_(std::move(api)), limits_(limits), port_(port), gidIndex_(gidIndex) {
  sendCq_ = api_->createCq(ctx, limits.maxCqSize, nullptr, nullptr, 0);
  if (sendCq_ == nullptr) throw IbError("ibv_create_cq (send) failed", errno);
  recvCq_ = api_->createCq(ctx, std::max(limits.maxRecvWr, 1), nullptr, nullptr, 0);
  if (recvCq_ == nullptr) {
    const int e = errno;
    (void)api_->destroyCq(sendCq_);
    throw IbError("ibv_create_cq (recv) failed", e);
  }
  ibv_qp_init_attr init{};
  init.send_cq = sendCq_;
  init.recv_cq = recvCq_;
  init.qp_type = IBV_QPT_RC;
  init.sq_sig_all = 0;
  init.cap.max_send_wr = limits.maxSendWr;
  init.cap.max_recv_wr = limits.maxRecvWr;
  init.cap.max_send_sge = 1;
  init.cap.max_recv_sge = 1;
  init.cap.max_inline_data = 0;
  qp_ = api_->createQp(pd, &init);
  if (qp_ == nullptr) {
    const int e = errno;
    (void)api_->destroyCq(recvCq_);
    (void)api_->destroyCq(sendCq_);
    throw IbError("ibv_create_qp failed", e);
  }

  // from here on a failure has to give back what exists already: the destructor does not run for a constructor that throws
  auto fail = [this](const std::string& what, int err) {
    (void)api_->destroyQp(qp_);
    (void)api_->destroyCq(recvCq_);
    (void)api_->destroyCq(sendCq_);
    qp_ = nullptr;
    sendCq_ = recvCq_ = nullptr;
    throw IbError(what, err);
  };
  ibv_port_attr pa{};
  if (api_->queryPort(ctx, static_cast<uint8_t>(port), &pa) != 0) fail("ibv_query_port failed", errno);
  info_.lid = pa.lid;
  info_.port = static_cast<uint8_t>(port);
  info_.linkLayer = pa.link_layer;
  info_.qpn = qp_->qp_num;
  info_.mtu = static_cast<int32_t>(pa.active_mtu);
  info_.useGrh = (pa.link_layer == IBV_LINK_LAYER_ETHERNET || gidIndex >= 0) ? 1 : 0;
  if (info_.useGrh) {
    ibv_gid gid{};
    if (api_->queryGid(ctx, static_cast<uint8_t>(port), std::max(gidIndex, 0), &gid) != 0) fail("ibv_query_gid failed", errno);
    info_.subnetPrefix = gid.global.subnet_prefix;
    info_.interfaceId = gid.global.interface_id;
  }

  ibv_qp_attr attr{};
  attr.qp_state = IBV_QPS_INIT;
  attr.pkey_index = 0;
  attr.port_num = static_cast<uint8_t>(port);
  attr.qp_access_flags = kMrAccess;
  if (api_->modifyQp(qp_, &attr, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0) {
    fail("ibv_modify_qp to INIT failed", errno);
  }

  sendWrs_.resize(limits.maxWrPerSend);
  sendSges_.resize(limits.maxWrPerSend);
  recvWrs_.resize(std::max(limits.maxRecvWr, 1));
  sendWcs_.resize(limits.maxCqPollNum);
  recvWcs_.resize(std::max(limits.maxRecvWr, 1));
}

IbQp::~IbQp() {
  if (qp_ != nullptr) (void)api_->destroyQp(qp_);
  if (recvCq_ != nullptr) (void)api_->destroyCq(recvCq_);
  if (sendCq_ != nullptr) (void)api_->destroyCq(sendCq_);
}

void IbQp::rtr(const IbQpInfo& remote) {
  ibv_qp_attr attr{};
  attr.qp_state = IBV_QPS_RTR;
  attr.path_mtu = static_cast<ibv_mtu>(std::min(info_.mtu, remote.mtu));
  attr.dest_qp_num = remote.qpn;
  attr.rq_psn = 0;
  attr.max_dest_rd_atomic = 1;
  attr.min_rnr_timer = 0x12;
  if (remote.useGrh || info_.useGrh) {
    attr.ah_attr.is_global = 1;
    attr.ah_attr.grh.dgid.global.subnet_prefix = remote.subnetPrefix;
    attr.ah_attr.grh.dgid.global.interface_id = remote.interfaceId;
    attr.ah_attr.grh.flow_label = 0;
    attr.ah_attr.grh.sgid_index = static_cast<uint8_t>(std::max(gidIndex_, 0));
    attr.ah_attr.grh.hop_limit = 255;
    attr.ah_attr.grh.traffic_class = 0;
  }
  attr.ah_attr.dlid = remote.lid;
  attr.ah_attr.sl = 0;
  attr.ah_attr.src_path_bits = 0;
  attr.ah_attr.port_num = static_cast<uint8_t>(port_);
  const int mask = IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC |
                   IBV_QP_MIN_RNR_TIMER;
  if (api_->modifyQp(qp_, &attr, mask) != 0) throw IbError("ibv_modify_qp to RTR failed", errno);
}

void IbQp::rts() {
  ibv_qp_attr attr{};
  attr.qp_state = IBV_QPS_RTS;
  attr.timeout = 18;
  attr.retry_cnt = 7;
  attr.rnr_retry = 7;
  attr.sq_psn = 0;
  attr.max_rd_atomic = 1;
  const int mask = IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC;
  if (api_->modifyQp(qp_, &attr, mask) != 0) throw IbError("ibv_modify_qp to RTS failed", errno);
}

ibv_send_wr& IbQp::nextSendWr(ibv_sge*& sge) {
  if (numStaged_ >= sendWrs_.size()) {
    throw Error("more than " + std::to_string(sendWrs_.size()) + " work requests staged without a postSend()", ErrorCode::InvalidUsage);
  }
  ibv_send_wr& wr = sendWrs_[numStaged_];
  sge = &sendSges_[numStaged_];
  std::memset(&wr, 0, sizeof(wr));
  std::memset(sge, 0, sizeof(*sge));
  wr.sg_list = sge;
  wr.num_sge = 1;
  wr.next = nullptr;
  if (numStaged_ > 0) sendWrs_[numStaged_ - 1].next = &wr;
  numStaged_++;
  return wr;
}

void IbQp::stageWrite(const IbMr& src, const IbMrInfo& dst, uint32_t size, uint64_t wrId, uint64_t srcOffset, uint64_t dstOffset,
                      bool signaled) {
  stageWriteWithImm(&src, dst, size, wrId, srcOffset, dstOffset, signaled, 0);
  sendWrs_[numStaged_ - 1].opcode = IBV_WR_RDMA_WRITE;
}

void IbQp::stageWriteWithImm(const IbMr* src, const IbMrInfo& dst, uint32_t size, uint64_t wrId, uint64_t srcOffset,
                             uint64_t dstOffset, bool signaled, uint32_t imm) {
  ibv_sge* sge;
  ibv_send_wr& wr = nextSendWr(sge);
  wr.wr_id = wrId;
  wr.opcode = IBV_WR_RDMA_WRITE_WITH_IMM;
  wr.send_flags = signaled ? IBV_SEND_SIGNALED : 0;
  wr.imm_data = imm;
  wr.wr.rdma.remote_addr = dst.addr + dstOffset;
  wr.wr.rdma.rkey = dst.rkey;
  if (src != nullptr && size != 0) {
    sge->addr = reinterpret_cast<uint64_t>(src->buff()) + srcOffset;
    sge->length = size;
    sge->lkey = src->lkey();
  } else {
    wr.sg_list = nullptr;  // a notification: no payload
    wr.num_sge = 0;
  }
  if (signaled) stagedSignaled_++;
}

void IbQp::stageAtomicAdd(const IbMr& landing, const IbMrInfo& dst, uint64_t wrId, uint64_t dstOffset, uint64_t add, bool signaled) {
  ibv_sge* sge;
  ibv_send_wr& wr = nextSendWr(sge);
  wr.wr_id = wrId;
  wr.opcode = IBV_WR_ATOMIC_FETCH_AND_ADD;
  wr.send_flags = signaled ? IBV_SEND_SIGNALED : 0;
  wr.wr.atomic.remote_addr = dst.addr + dstOffset;
  wr.wr.atomic.rkey = dst.rkey;
  wr.wr.atomic.compare_add = add;
  sge->addr = reinterpret_cast<uint64_t>(landing.buff());
  sge->length = sizeof(uint64_t);
  sge->lkey = landing.lkey();
  if (signaled) stagedSignaled_++;
}

void IbQp::postSend() {
  if (numStaged_ == 0) return;
  ibv_send_wr* bad = nullptr;
  const int rc = api_->postSend(qp_, sendWrs_.data(), &bad);
  const size_t staged = numStaged_;
  numStaged_ = 0;
  if (rc != 0) {
    stagedSignaled_ = 0;
    throw IbError("ibv_post_send failed for a chain of " + std::to_string(staged) + " work requests", rc);
  }
  outstandingSignaled_ += stagedSignaled_;
  stagedSignaled_ = 0;
}

void IbQp::stageRecv(uint64_t wrId) {
  if (numStagedRecv_ >= recvWrs_.size()) throw Error("too many receive work requests staged", ErrorCode::InvalidUsage);
  ibv_recv_wr& wr = recvWrs_[numStagedRecv_];
  std::memset(&wr, 0, sizeof(wr));
  wr.wr_id = wrId;
  if (numStagedRecv_ > 0) recvWrs_[numStagedRecv_ - 1].next = &wr;
  numStagedRecv_++;
}

void IbQp::postRecv() {
  if (numStagedRecv_ == 0) return;
  ibv_recv_wr* bad = nullptr;
  const int rc = api_->postRecv(qp_, recvWrs_.data(), &bad);
  numStagedRecv_ = 0;
  if (rc != 0) throw IbError("ibv_post_recv failed", rc);
}

int IbQp::pollSendCq() {
  const int n = api_->pollCq(sendCq_, static_cast<int>(sendWcs_.size()), sendWcs_.data());
  if (n > 0) outstandingSignaled_ = std::max(0, outstandingSignaled_ - n);  // error completions also come for unsignalled requests
  return n;
}

int IbQp::pollRecvCq() { return api_->pollCq(recvCq_, static_cast<int>(recvWcs_.size()), recvWcs_.data()); }

std::string IbQp::wcStatusString(int status) const {
  if (api_->wcStatusStr != nullptr) {
    const char* s = api_->wcStatusStr(status);
    if (s != nullptr) return s;
  }
  return "work completion status " + std::to_string(status);
}

// ------------------------------------------------------------------------------------------ IbCtx
IbCtx::IbCtx(const std::string& deviceName) : api_(IbvApi::get()), deviceName_(deviceName) {
  int n = 0;
  ibv_device** list = api_->getDeviceList(&n);
  if (list == nullptr) throw IbError("ibv_get_device_list failed", errno);
  for (int i = 0; i < n && ctx_ == nullptr; i++) {
    if (deviceName == api_->getDeviceName(list[i])) ctx_ = api_->openDevice(list[i]);
  }
  const int e = errno;
  api_->freeDeviceList(list);
  if (ctx_ == nullptr) throw IbError("cannot open InfiniBand device '" + deviceName + "'", e);
  pd_ = api_->allocPd(ctx_);
  if (pd_ == nullptr) {
    const int e2 = errno;
    (void)api_->closeDevice(ctx_);
    ctx_ = nullptr;
    throw IbError("ibv_alloc_pd failed on " + deviceName, e2);
  }
  ibv_device_attr da{};
  if (api_->queryDevice(ctx_, &da) == 0) {
    numPorts_ = da.phys_port_cnt;
    atomics_ = da.atomic_cap != IBV_ATOMIC_NONE;
  }
  virtualFunction_ = ::access(("/sys/class/infiniband/" + deviceName + "/device/physfn").c_str(), F_OK) == 0;
}

IbCtx::~IbCtx() {
  if (pd_ != nullptr) (void)api_->deallocPd(pd_);
  if (ctx_ != nullptr) (void)api_->closeDevice(ctx_);
}

bool IbCtx::isPortUsable(int port, int gidIndex) const {
  ibv_port_attr pa{};
  if (api_->queryPort(ctx_, static_cast<uint8_t>(port), &pa) != 0) return false;
  if (pa.state != IBV_PORT_ACTIVE) return false;
  if (pa.link_layer != IBV_LINK_LAYER_ETHERNET && pa.link_layer != IBV_LINK_LAYER_INFINIBAND &&
      pa.link_layer != IBV_LINK_LAYER_UNSPECIFIED) {
    return false;
  }
  const int needGid = pa.link_layer == IBV_LINK_LAYER_ETHERNET ? std::max(gidIndex, 0) : gidIndex;
  return needGid < 0 || needGid < pa.gid_tbl_len;
}

int IbCtx::anyUsablePort(int gidIndex) const {
  for (int p = 1; p <= numPorts_; p++) {
    if (isPortUsable(p, gidIndex)) return p;
  }
  return -1;
}

std::shared_ptr<IbQp> IbCtx::createQp(int port, int gidIndex, const IbQp::Limits& limits) {
  if (gidIndex < 0) gidIndex = env()->ibGidIndex;
  if (port < 0) {
    port = anyUsablePort(gidIndex);
    if (port < 0) throw Error("no usable port on InfiniBand device " + deviceName_, ErrorCode::InvalidUsage);
  } else if (!isPortUsable(port, gidIndex)) {
    throw Error("port " + std::to_string(port) + " of " + deviceName_ + " is not usable", ErrorCode::InvalidUsage);
  }
  return std::make_shared<IbQp>(api_, ctx_, pd_, port, gidIndex, limits);
}

std::shared_ptr<const IbMr> IbCtx::registerMr(void* buff, size_t size) { return std::make_shared<const IbMr>(api_, pd_, buff, size); }

}  // namespace mscclpp
