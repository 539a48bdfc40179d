// InfiniBand verbs layer: the run-time loaded function table, device contexts, memory regions and reliable-connection
// queue pairs that IBConnection (connection.cc) is built on. Same roles as the reference's IbCtx / IbQp / IbMr
// (src/core/include/ib.hpp:25-177, src/core/ib.cc:70-325, src/core/ibverbs_wrapper.cc:30-110).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include <mscclpp/core.hpp>

#include "ib_verbs_abi.hpp"

namespace mscclpp {

// libibverbs (or a provider with the same entry points), loaded with dlopen. MSCCLPP_IBV_SO names the library; the
// default is libibverbs.so.1. Nothing of it is linked, so the core library loads on machines without rdma-core.
struct IbvApi {
  // The process-wide table; throws Error(SystemError) when the library or one of its required symbols is missing.
  static std::shared_ptr<const IbvApi> get();
  // True when get() would succeed.
  static bool available();

  ibv_device** (*getDeviceList)(int*) = nullptr;
  void (*freeDeviceList)(ibv_device**) = nullptr;
  const char* (*getDeviceName)(ibv_device*) = nullptr;
  ibv_context* (*openDevice)(ibv_device*) = nullptr;
  int (*closeDevice)(ibv_context*) = nullptr;
  int (*queryDevice)(ibv_context*, ibv_device_attr*) = nullptr;
  int (*queryPort)(ibv_context*, uint8_t, ibv_port_attr*) = nullptr;
  int (*queryGid)(ibv_context*, uint8_t, int, ibv_gid*) = nullptr;
  ibv_pd* (*allocPd)(ibv_context*) = nullptr;
  int (*deallocPd)(ibv_pd*) = nullptr;
  ibv_mr* (*regMr)(ibv_pd*, void*, size_t, int) = nullptr;
  ibv_mr* (*regDmabufMr)(ibv_pd*, uint64_t, size_t, uint64_t, int, int) = nullptr;  // optional
  int (*deregMr)(ibv_mr*) = nullptr;
  ibv_cq* (*createCq)(ibv_context*, int, void*, ibv_comp_channel*, int) = nullptr;
  int (*destroyCq)(ibv_cq*) = nullptr;
  ibv_qp* (*createQp)(ibv_pd*, ibv_qp_init_attr*) = nullptr;
  int (*modifyQp)(ibv_qp*, ibv_qp_attr*, int) = nullptr;
  int (*destroyQp)(ibv_qp*) = nullptr;
  const char* (*wcStatusStr)(int) = nullptr;  // optional

  // Fast path. libibverbs does not export these: its header calls them through the device context's table. A provider
  // that does export them (the software provider of the tests) is called directly.
  int postSend(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) const;
  int postRecv(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad) const;
  int pollCq(ibv_cq* cq, int n, ibv_wc* wc) const;

  std::string path;

 private:
  int (*postSendSym_)(ibv_qp*, ibv_send_wr*, ibv_send_wr**) = nullptr;
  int (*postRecvSym_)(ibv_qp*, ibv_recv_wr*, ibv_recv_wr**) = nullptr;
  int (*pollCqSym_)(ibv_cq*, int, ibv_wc*) = nullptr;
  void* handle_ = nullptr;
  friend struct IbvApiLoader;
};

// What a peer needs to write into a registered region.
struct IbMrInfo {
  uint64_t addr = 0;
  uint32_t rkey = 0;
};

class IbMr {
 public:
  IbMr(std::shared_ptr<const IbvApi> api, ibv_pd* pd, void* buff, size_t size);
  ~IbMr();
  IbMr(const IbMr&) = delete;
  IbMr& operator=(const IbMr&) = delete;
  IbMrInfo info() const;
  uint32_t lkey() const;
  void* buff() const { return buff_; }
  size_t size() const { return size_; }
  bool viaDmabuf() const { return dmabuf_; }

 private:
  std::shared_ptr<const IbvApi> api_;
  ibv_mr* mr_ = nullptr;
  void* buff_;
  size_t size_;
  bool dmabuf_ = false;
};

// What a peer needs to connect its queue pair to this one.
struct IbQpInfo {
  uint16_t lid = 0;
  uint8_t port = 0;
  uint8_t linkLayer = 0;
  uint32_t qpn = 0;
  uint64_t subnetPrefix = 0;  // of the GID at gidIndex (network byte order, as the device reports it)
  uint64_t interfaceId = 0;
  int32_t mtu = 0;            // ibv_mtu of the port
  uint8_t useGrh = 0;         // RoCE, or an explicit GID index on InfiniBand
};

class IbQp {
 public:
  struct Limits {
    int maxCqSize;
    int maxCqPollNum;
    int maxSendWr;
    int maxRecvWr;
    int maxWrPerSend;
  };
  IbQp(std::shared_ptr<const IbvApi> api, ibv_context* ctx, ibv_pd* pd, int port, int gidIndex, const Limits& limits);
  ~IbQp();
  IbQp(const IbQp&) = delete;
  IbQp& operator=(const IbQp&) = delete;

  const IbQpInfo& info() const { return info_; }
  // RESET -> INIT happened in the constructor; these take the pair to ready-to-receive and ready-to-send.
  void rtr(const IbQpInfo& remote);
  void rts();

  // Work requests are staged (up to maxWrPerSend) and handed to the device as one chain by postSend().
  void stageWrite(const IbMr& src, const IbMrInfo& dst, uint32_t size, uint64_t wrId, uint64_t srcOffset, uint64_t dstOffset,
                  bool signaled);
  void stageWriteWithImm(const IbMr* src, const IbMrInfo& dst, uint32_t size, uint64_t wrId, uint64_t srcOffset,
                         uint64_t dstOffset, bool signaled, uint32_t imm);
  // fetch-and-add of `add` on the 8 bytes at dst + dstOffset; the old value lands in `landing` (8 bytes of local memory)
  void stageAtomicAdd(const IbMr& landing, const IbMrInfo& dst, uint64_t wrId, uint64_t dstOffset, uint64_t add, bool signaled);
  int numStaged() const { return static_cast<int>(numStaged_); }
  void postSend();

  void stageRecv(uint64_t wrId);
  void postRecv();

  // Polls up to maxCqPollNum completions; they stay readable through sendWc()/recvWc() until the next poll. Returns
  // their number, negative on a device error.
  int pollSendCq();
  int pollRecvCq();
  const ibv_wc& sendWc(int i) const { return sendWcs_[i]; }
  const ibv_wc& recvWc(int i) const { return recvWcs_[i]; }
  std::string wcStatusString(int status) const;
  // signaled send work requests posted and not yet polled
  int outstandingSignaled() const { return outstandingSignaled_; }

 private:
  ibv_send_wr& nextSendWr(ibv_sge*& sge);

  std::shared_ptr<const IbvApi> api_;
  Limits limits_;
  int port_;
  int gidIndex_;
  IbQpInfo info_;
  ibv_qp* qp_ = nullptr;
  ibv_cq* sendCq_ = nullptr;
  ibv_cq* recvCq_ = nullptr;
  std::vector<ibv_send_wr> sendWrs_;
  std::vector<ibv_sge> sendSges_;
  std::vector<ibv_recv_wr> recvWrs_;
  std::vector<ibv_wc> sendWcs_;
  std::vector<ibv_wc> recvWcs_;
  size_t numStaged_ = 0;
  size_t numStagedRecv_ = 0;
  int stagedSignaled_ = 0;
  int outstandingSignaled_ = 0;
};

class IbCtx {
 public:
  explicit IbCtx(const std::string& deviceName);
  ~IbCtx();
  IbCtx(const IbCtx&) = delete;
  IbCtx& operator=(const IbCtx&) = delete;

  const std::string& deviceName() const { return deviceName_; }
  // port < 0: the first active port that has the requested GID index (index < 0: none needed on InfiniBand, 0 on RoCE)
  std::shared_ptr<IbQp> createQp(int port, int gidIndex, const IbQp::Limits& limits);
  std::shared_ptr<const IbMr> registerMr(void* buff, size_t size);
  bool supportsRdmaAtomics() const { return atomics_; }
  bool isMlx5() const { return deviceName_.rfind("mlx5", 0) == 0; }
  // SR-IOV virtual function (sysfs: the device has a physfn link)
  bool isVirtualFunction() const { return virtualFunction_; }
  bool isPortUsable(int port, int gidIndex) const;
  int anyUsablePort(int gidIndex) const;

 private:
  std::shared_ptr<const IbvApi> api_;
  std::string deviceName_;
  ibv_context* ctx_ = nullptr;
  ibv_pd* pd_ = nullptr;
  int numPorts_ = 0;
  bool atomics_ = false;
  bool virtualFunction_ = false;
};

// Device names as the loaded library lists them (MSCCLPP_HCA_DEVICES filters and orders them); empty when the library
// cannot be loaded.
std::vector<std::string> ibDeviceNamesFromLibrary();

}  // namespace mscclpp
