// A software provider of the verbs entry points that the InfiniBand transport uses, for tests on machines without an
// HCA: two devices ("fake0", "fake1") whose queue pairs live in one process. RDMA writes are memcpy, fetch-and-add is
// an atomic on the target word, write-with-immediate consumes a posted receive of the destination queue pair. It checks
// what a device checks (queue-pair state transitions and their attribute masks, local and remote keys and ranges,
// receive-queue underrun) and answers with the matching error completions, so that the transport's sequencing and error
// paths are exercised. Knobs, read at call time:
//   FAKE_IBV_NO_ATOMICS=1        devices report no RDMA atomics
//   FAKE_IBV_ROCE=1              ports report an Ethernet link layer (GIDs required)
//   FAKE_IBV_DROP_COMPLETIONS=1  successful send completions are not delivered (a flush then runs into its time limit)
// Build: g++ -shared -fPIC -DMSCCLPP_IB_OWN_ABI -I <csrc> fake_ibverbs.cc -o libfake_ibverbs.so
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>

#include "core/ib_verbs_abi.hpp"

extern "C" {
struct ibv_device {
  char name[64];
  int index;
};
}

namespace {

bool knob(const char* name) {
  const char* v = std::getenv(name);
  return v != nullptr && v[0] != '\0' && v[0] != '0';
}

struct FakeCq {
  ibv_cq base;
  std::deque<ibv_wc> q;
};

struct FakeQp {
  ibv_qp base;
  uint32_t destQpn = 0;
  std::deque<uint64_t> recvs;  // wr_ids of posted receives
};

struct FakeMr {
  ibv_mr base;
};

std::mutex g_mutex;
ibv_device g_devices[2] = {{"fake0", 0}, {"fake1", 1}};
std::map<uint32_t, FakeMr*> g_mrs;  // key (lkey == rkey) -> region
std::map<uint32_t, FakeQp*> g_qps;  // qp number -> queue pair
uint32_t g_nextKey = 0x1000;
uint32_t g_nextQpn = 0x40;

bool inRegion(uint32_t key, uint64_t addr, uint64_t len) {
  auto it = g_mrs.find(key);
  if (it == g_mrs.end()) return false;
  const uint64_t base = reinterpret_cast<uint64_t>(it->second->base.addr);
  return addr >= base && addr + len <= base + it->second->base.length;
}

void complete(ibv_cq* cq, uint64_t wrId, ibv_wc_status status, ibv_wc_opcode op, uint32_t qpn, uint32_t imm = 0, bool withImm = false) {
  ibv_wc wc{};
  wc.wr_id = wrId;
  wc.status = status;
  wc.opcode = op;
  wc.qp_num = qpn;
  wc.imm_data = imm;
  wc.wc_flags = withImm ? IBV_WC_WITH_IMM : 0;
  reinterpret_cast<FakeCq*>(cq)->q.push_back(wc);
}

int fakePostSend(ibv_qp* q, ibv_send_wr* wr, ibv_send_wr** bad) {
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeQp* qp = reinterpret_cast<FakeQp*>(q);
  if (qp->base.state != IBV_QPS_RTS && qp->base.state != IBV_QPS_ERR) {
    if (bad) *bad = wr;
    return EINVAL;
  }
  for (; wr != nullptr; wr = wr->next) {
    ibv_wc_opcode op = wr->opcode == IBV_WR_ATOMIC_FETCH_AND_ADD ? IBV_WC_FETCH_ADD : IBV_WC_RDMA_WRITE;
    if (qp->base.state == IBV_QPS_ERR) {  // after an error everything is flushed
      complete(qp->base.send_cq, wr->wr_id, IBV_WC_WR_FLUSH_ERR, op, qp->base.qp_num);
      continue;
    }
    ibv_wc_status status = IBV_WC_SUCCESS;
    const uint64_t localLen = wr->num_sge > 0 ? wr->sg_list[0].length : 0;
    FakeQp* peer = nullptr;
    auto it = g_qps.find(qp->destQpn);
    if (it != g_qps.end()) peer = it->second;
    if (wr->num_sge > 1) {
      status = IBV_WC_LOC_LEN_ERR;
    } else if (localLen > 0 && !inRegion(wr->sg_list[0].lkey, wr->sg_list[0].addr, localLen)) {
      status = IBV_WC_LOC_PROT_ERR;
    } else if (peer == nullptr || (peer->base.state != IBV_QPS_RTR && peer->base.state != IBV_QPS_RTS) || peer->destQpn != qp->base.qp_num) {
      status = IBV_WC_RETRY_EXC_ERR;
    } else if (wr->opcode == IBV_WR_RDMA_WRITE || wr->opcode == IBV_WR_RDMA_WRITE_WITH_IMM) {
      if (localLen > 0 && !inRegion(wr->wr.rdma.rkey, wr->wr.rdma.remote_addr, localLen)) {
        status = IBV_WC_REM_ACCESS_ERR;
      } else if (wr->opcode == IBV_WR_RDMA_WRITE_WITH_IMM && peer->recvs.empty()) {
        status = IBV_WC_RNR_RETRY_EXC_ERR;
      } else {
        if (localLen > 0) std::memcpy(reinterpret_cast<void*>(wr->wr.rdma.remote_addr), reinterpret_cast<void*>(wr->sg_list[0].addr), localLen);
        if (wr->opcode == IBV_WR_RDMA_WRITE_WITH_IMM) {
          const uint64_t recvId = peer->recvs.front();
          peer->recvs.pop_front();
          complete(peer->base.recv_cq, recvId, IBV_WC_SUCCESS, IBV_WC_RECV_RDMA_WITH_IMM, peer->base.qp_num, wr->imm_data, true);
        }
      }
    } else if (wr->opcode == IBV_WR_ATOMIC_FETCH_AND_ADD) {
      if (localLen != 8 || (wr->wr.atomic.remote_addr & 7) != 0 || !inRegion(wr->wr.atomic.rkey, wr->wr.atomic.remote_addr, 8)) {
        status = IBV_WC_REM_ACCESS_ERR;
      } else {
        const uint64_t old = __atomic_fetch_add(reinterpret_cast<uint64_t*>(wr->wr.atomic.remote_addr), wr->wr.atomic.compare_add, __ATOMIC_SEQ_CST);
        std::memcpy(reinterpret_cast<void*>(wr->sg_list[0].addr), &old, 8);
      }
    } else {
      status = IBV_WC_LOC_QP_OP_ERR;
    }
    if (status != IBV_WC_SUCCESS) {
      qp->base.state = IBV_QPS_ERR;
      complete(qp->base.send_cq, wr->wr_id, status, op, qp->base.qp_num);
    } else if ((wr->send_flags & IBV_SEND_SIGNALED) && !knob("FAKE_IBV_DROP_COMPLETIONS")) {
      complete(qp->base.send_cq, wr->wr_id, IBV_WC_SUCCESS, op, qp->base.qp_num);
    }
  }
  return 0;
}

int fakePostRecv(ibv_qp* q, ibv_recv_wr* wr, ibv_recv_wr** bad) {
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeQp* qp = reinterpret_cast<FakeQp*>(q);
  if (qp->base.state == IBV_QPS_RESET) {
    if (bad) *bad = wr;
    return EINVAL;
  }
  for (; wr != nullptr; wr = wr->next) qp->recvs.push_back(wr->wr_id);
  return 0;
}

int fakePollCq(ibv_cq* c, int n, ibv_wc* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeCq* cq = reinterpret_cast<FakeCq*>(c);
  int got = 0;
  while (got < n && !cq->q.empty()) {
    out[got++] = cq->q.front();
    cq->q.pop_front();
  }
  return got;
}

}  // namespace

extern "C" {

ibv_device** ibv_get_device_list(int* n) {
  ibv_device** list = static_cast<ibv_device**>(std::calloc(3, sizeof(ibv_device*)));
  list[0] = &g_devices[0];
  list[1] = &g_devices[1];
  if (n) *n = 2;
  return list;
}
void ibv_free_device_list(ibv_device** list) { std::free(list); }
const char* ibv_get_device_name(ibv_device* d) { return d->name; }

ibv_context* ibv_open_device(ibv_device* d) {
  ibv_context* ctx = static_cast<ibv_context*>(std::calloc(1, sizeof(ibv_context)));
  ctx->device = d;
  ctx->ops.post_send = fakePostSend;
  ctx->ops.post_recv = fakePostRecv;
  ctx->ops.poll_cq = fakePollCq;
  return ctx;
}
int ibv_close_device(ibv_context* ctx) {
  std::free(ctx);
  return 0;
}

int ibv_query_device(ibv_context*, ibv_device_attr* attr) {
  std::memset(attr, 0, sizeof(*attr));
  attr->phys_port_cnt = 1;
  attr->atomic_cap = knob("FAKE_IBV_NO_ATOMICS") ? IBV_ATOMIC_NONE : IBV_ATOMIC_HCA;
  attr->max_qp_wr = 16384;
  return 0;
}

int ibv_query_port(ibv_context* ctx, uint8_t port, ibv_port_attr* attr) {
  if (port != 1) return EINVAL;
  std::memset(attr, 0, sizeof(*attr));
  attr->state = IBV_PORT_ACTIVE;
  attr->max_mtu = IBV_MTU_4096;
  attr->active_mtu = ctx->device->index == 0 ? IBV_MTU_4096 : IBV_MTU_2048;  // the pair must settle on the smaller one
  attr->gid_tbl_len = 4;
  attr->lid = static_cast<uint16_t>(1 + ctx->device->index);
  attr->link_layer = knob("FAKE_IBV_ROCE") ? IBV_LINK_LAYER_ETHERNET : IBV_LINK_LAYER_INFINIBAND;
  return 0;
}

int ibv_query_gid(ibv_context* ctx, uint8_t port, int index, ibv_gid* gid) {
  if (port != 1 || index < 0 || index >= 4) return EINVAL;
  gid->global.subnet_prefix = 0xfe80000000000000ull;
  gid->global.interface_id = 0x1000u + 16u * ctx->device->index + index;
  return 0;
}

ibv_pd* ibv_alloc_pd(ibv_context* ctx) {
  ibv_pd* pd = static_cast<ibv_pd*>(std::calloc(1, sizeof(ibv_pd)));
  pd->context = ctx;
  return pd;
}
int ibv_dealloc_pd(ibv_pd* pd) {
  std::free(pd);
  return 0;
}

ibv_mr* ibv_reg_mr(ibv_pd* pd, void* addr, size_t length, int access) {
  if (addr == nullptr || length == 0 || (access & IBV_ACCESS_LOCAL_WRITE) == 0) {
    errno = EINVAL;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeMr* mr = new FakeMr();
  mr->base.context = pd->context;
  mr->base.pd = pd;
  mr->base.addr = addr;
  mr->base.length = length;
  mr->base.lkey = mr->base.rkey = g_nextKey++;
  g_mrs[mr->base.lkey] = mr;
  return &mr->base;
}
int ibv_dereg_mr(ibv_mr* m) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_mrs.erase(m->lkey);
  delete reinterpret_cast<FakeMr*>(m);
  return 0;
}

ibv_cq* ibv_create_cq(ibv_context* ctx, int cqe, void*, ibv_comp_channel*, int) {
  if (cqe <= 0) {
    errno = EINVAL;
    return nullptr;
  }
  FakeCq* cq = new FakeCq();
  cq->base.context = ctx;
  cq->base.cqe = cqe;
  return &cq->base;
}
int ibv_destroy_cq(ibv_cq* cq) {
  delete reinterpret_cast<FakeCq*>(cq);
  return 0;
}

ibv_qp* ibv_create_qp(ibv_pd* pd, ibv_qp_init_attr* init) {
  if (init->qp_type != IBV_QPT_RC || init->send_cq == nullptr || init->recv_cq == nullptr || init->cap.max_send_wr == 0) {
    errno = EINVAL;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeQp* qp = new FakeQp();
  qp->base.context = pd->context;
  qp->base.pd = pd;
  qp->base.send_cq = init->send_cq;
  qp->base.recv_cq = init->recv_cq;
  qp->base.qp_num = g_nextQpn++;
  qp->base.state = IBV_QPS_RESET;
  qp->base.qp_type = IBV_QPT_RC;
  g_qps[qp->base.qp_num] = qp;
  return &qp->base;
}
int ibv_destroy_qp(ibv_qp* q) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_qps.erase(q->qp_num);
  delete reinterpret_cast<FakeQp*>(q);
  return 0;
}

int ibv_modify_qp(ibv_qp* q, ibv_qp_attr* attr, int mask) {
  std::lock_guard<std::mutex> lock(g_mutex);
  FakeQp* qp = reinterpret_cast<FakeQp*>(q);
  if ((mask & IBV_QP_STATE) == 0) return EINVAL;
  const int needInit = IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS;
  const int needRtr = IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
  const int needRts = IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC;
  switch (attr->qp_state) {
    case IBV_QPS_INIT:
      if (qp->base.state != IBV_QPS_RESET || (mask & needInit) != needInit || attr->port_num != 1) return EINVAL;
      break;
    case IBV_QPS_RTR:
      if (qp->base.state != IBV_QPS_INIT || (mask & needRtr) != needRtr) return EINVAL;
      if (attr->path_mtu < IBV_MTU_256 || attr->path_mtu > IBV_MTU_2048) return EINVAL;  // fake1's port runs at 2048
      if (knob("FAKE_IBV_ROCE") && !attr->ah_attr.is_global) return EINVAL;
      if (attr->ah_attr.is_global && attr->ah_attr.grh.dgid.global.subnet_prefix != 0xfe80000000000000ull) return EINVAL;
      qp->destQpn = attr->dest_qp_num;
      break;
    case IBV_QPS_RTS:
      if (qp->base.state != IBV_QPS_RTR || (mask & needRts) != needRts) return EINVAL;
      break;
    default:
      return EINVAL;
  }
  qp->base.state = attr->qp_state;
  return 0;
}

// libibverbs does not export the fast-path calls (its header reaches them through the context's table). Built with
// -DFAKE_IBV_NO_FASTPATH_SYMBOLS this provider does not either, which exercises that route of the loader.
#if !defined(FAKE_IBV_NO_FASTPATH_SYMBOLS)
int ibv_post_send(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) { return fakePostSend(qp, wr, bad); }
int ibv_post_recv(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad) { return fakePostRecv(qp, wr, bad); }
int ibv_poll_cq(ibv_cq* cq, int n, ibv_wc* wc) { return fakePollCq(cq, n, wc); }
#endif

const char* ibv_wc_status_str(int status) {
  switch (status) {
    case IBV_WC_SUCCESS:
      return "success";
    case IBV_WC_LOC_PROT_ERR:
      return "local protection error";
    case IBV_WC_WR_FLUSH_ERR:
      return "work request flushed";
    case IBV_WC_REM_ACCESS_ERR:
      return "remote access error";
    case IBV_WC_RETRY_EXC_ERR:
      return "transport retry counter exceeded";
    case IBV_WC_RNR_RETRY_EXC_ERR:
      return "receiver-not-ready retry counter exceeded";
    default:
      return "other error";
  }
}

}  // extern "C"
