// The slice of the verbs ABI (rdma-core's public <infiniband/verbs.h>) that the InfiniBand transport uses.
// When that header is installed it is used as is. Otherwise the declarations below stand in for it: the same type, field
// and constant names, in the layout of libibverbs' stable 1.x ABI, so that the transport can be built and tested (against
// a software provider, tests/cpp/fake_ibverbs.cc) on machines without rdma-core. Only what ib.cc touches is declared.
// The library itself is never linked: it is loaded at run time (MSCCLPP_IBV_SO, default libibverbs.so.1), as the
// reference does (src/core/ibverbs_wrapper.cc:30-110).
#pragma once

#if defined(__has_include)
#if __has_include(<infiniband/verbs.h>) && !defined(MSCCLPP_IB_OWN_ABI)
#define MSCCLPP_IB_SYSTEM_HEADER 1
#endif
#endif

#if defined(MSCCLPP_IB_SYSTEM_HEADER)
#include <infiniband/verbs.h>
#else

#include <pthread.h>

#include <cstddef>
#include <cstdint>

extern "C" {

struct ibv_device;
struct ibv_context;
struct ibv_comp_channel;
struct ibv_srq;
struct ibv_ah;
struct ibv_mw;
struct ibv_mw_bind;

union ibv_gid {
  uint8_t raw[16];
  struct {
    uint64_t subnet_prefix;  // big endian
    uint64_t interface_id;   // big endian
  } global;
};

enum ibv_mtu { IBV_MTU_256 = 1, IBV_MTU_512 = 2, IBV_MTU_1024 = 3, IBV_MTU_2048 = 4, IBV_MTU_4096 = 5 };
enum ibv_port_state {
  IBV_PORT_NOP = 0,
  IBV_PORT_DOWN = 1,
  IBV_PORT_INIT = 2,
  IBV_PORT_ARMED = 3,
  IBV_PORT_ACTIVE = 4,
  IBV_PORT_ACTIVE_DEFER = 5
};
enum { IBV_LINK_LAYER_UNSPECIFIED = 0, IBV_LINK_LAYER_INFINIBAND = 1, IBV_LINK_LAYER_ETHERNET = 2 };
enum ibv_atomic_cap { IBV_ATOMIC_NONE = 0, IBV_ATOMIC_HCA = 1, IBV_ATOMIC_GLOB = 2 };

struct ibv_device_attr {
  char fw_ver[64];
  uint64_t node_guid;
  uint64_t sys_image_guid;
  uint64_t max_mr_size;
  uint64_t page_size_cap;
  uint32_t vendor_id;
  uint32_t vendor_part_id;
  uint32_t hw_ver;
  int max_qp;
  int max_qp_wr;
  unsigned int device_cap_flags;
  int max_sge;
  int max_sge_rd;
  int max_cq;
  int max_cqe;
  int max_mr;
  int max_pd;
  int max_qp_rd_atom;
  int max_ee_rd_atom;
  int max_res_rd_atom;
  int max_qp_init_rd_atom;
  int max_ee_init_rd_atom;
  enum ibv_atomic_cap atomic_cap;
  int max_ee;
  int max_rdd;
  int max_mw;
  int max_raw_ipv6_qp;
  int max_raw_ethy_qp;
  int max_mcast_grp;
  int max_mcast_qp_attach;
  int max_total_mcast_qp_attach;
  int max_ah;
  int max_fmr;
  int max_map_per_fmr;
  int max_srq;
  int max_srq_wr;
  int max_srq_sge;
  uint16_t max_pkeys;
  uint8_t local_ca_ack_delay;
  uint8_t phys_port_cnt;
};

struct ibv_port_attr {
  enum ibv_port_state state;
  enum ibv_mtu max_mtu;
  enum ibv_mtu active_mtu;
  int gid_tbl_len;
  uint32_t port_cap_flags;
  uint32_t max_msg_sz;
  uint32_t bad_pkey_cntr;
  uint32_t qkey_viol_cntr;
  uint16_t pkey_tbl_len;
  uint16_t lid;
  uint16_t sm_lid;
  uint8_t lmc;
  uint8_t max_vl_num;
  uint8_t sm_sl;
  uint8_t subnet_timeout;
  uint8_t init_type_reply;
  uint8_t active_width;
  uint8_t active_speed;
  uint8_t phys_state;
  uint8_t link_layer;
  uint8_t flags;
  uint16_t port_cap_flags2;
  uint32_t active_speed_ex;
};

struct ibv_pd {
  struct ibv_context* context;
  uint32_t handle;
};

struct ibv_mr {
  struct ibv_context* context;
  struct ibv_pd* pd;
  void* addr;
  size_t length;
  uint32_t handle;
  uint32_t lkey;
  uint32_t rkey;
};

enum ibv_access_flags {
  IBV_ACCESS_LOCAL_WRITE = 1,
  IBV_ACCESS_REMOTE_WRITE = 1 << 1,
  IBV_ACCESS_REMOTE_READ = 1 << 2,
  IBV_ACCESS_REMOTE_ATOMIC = 1 << 3,
  IBV_ACCESS_RELAXED_ORDERING = 1 << 20
};

struct ibv_global_route {
  union ibv_gid dgid;
  uint32_t flow_label;
  uint8_t sgid_index;
  uint8_t hop_limit;
  uint8_t traffic_class;
};

struct ibv_ah_attr {
  struct ibv_global_route grh;
  uint16_t dlid;
  uint8_t sl;
  uint8_t src_path_bits;
  uint8_t static_rate;
  uint8_t is_global;
  uint8_t port_num;
};

enum ibv_qp_type { IBV_QPT_RC = 2, IBV_QPT_UC = 3, IBV_QPT_UD = 4 };
enum ibv_qp_state {
  IBV_QPS_RESET = 0,
  IBV_QPS_INIT = 1,
  IBV_QPS_RTR = 2,
  IBV_QPS_RTS = 3,
  IBV_QPS_SQD = 4,
  IBV_QPS_SQE = 5,
  IBV_QPS_ERR = 6,
  IBV_QPS_UNKNOWN = 7
};
enum ibv_mig_state { IBV_MIG_MIGRATED = 0, IBV_MIG_REARM = 1, IBV_MIG_ARMED = 2 };

struct ibv_qp_cap {
  uint32_t max_send_wr;
  uint32_t max_recv_wr;
  uint32_t max_send_sge;
  uint32_t max_recv_sge;
  uint32_t max_inline_data;
};

struct ibv_cq {
  struct ibv_context* context;
  struct ibv_comp_channel* channel;
  void* cq_context;
  uint32_t handle;
  int cqe;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t comp_events_completed;
  uint32_t async_events_completed;
};

struct ibv_qp_init_attr {
  void* qp_context;
  struct ibv_cq* send_cq;
  struct ibv_cq* recv_cq;
  struct ibv_srq* srq;
  struct ibv_qp_cap cap;
  enum ibv_qp_type qp_type;
  int sq_sig_all;
};

struct ibv_qp_attr {
  enum ibv_qp_state qp_state;
  enum ibv_qp_state cur_qp_state;
  enum ibv_mtu path_mtu;
  enum ibv_mig_state path_mig_state;
  uint32_t qkey;
  uint32_t rq_psn;
  uint32_t sq_psn;
  uint32_t dest_qp_num;
  unsigned int qp_access_flags;
  struct ibv_qp_cap cap;
  struct ibv_ah_attr ah_attr;
  struct ibv_ah_attr alt_ah_attr;
  uint16_t pkey_index;
  uint16_t alt_pkey_index;
  uint8_t en_sqd_async_notify;
  uint8_t sq_draining;
  uint8_t max_rd_atomic;
  uint8_t max_dest_rd_atomic;
  uint8_t min_rnr_timer;
  uint8_t port_num;
  uint8_t timeout;
  uint8_t retry_cnt;
  uint8_t rnr_retry;
  uint8_t alt_port_num;
  uint8_t alt_timeout;
  uint32_t rate_limit;
};

enum ibv_qp_attr_mask {
  IBV_QP_STATE = 1 << 0,
  IBV_QP_CUR_STATE = 1 << 1,
  IBV_QP_EN_SQD_ASYNC_NOTIFY = 1 << 2,
  IBV_QP_ACCESS_FLAGS = 1 << 3,
  IBV_QP_PKEY_INDEX = 1 << 4,
  IBV_QP_PORT = 1 << 5,
  IBV_QP_QKEY = 1 << 6,
  IBV_QP_AV = 1 << 7,
  IBV_QP_PATH_MTU = 1 << 8,
  IBV_QP_TIMEOUT = 1 << 9,
  IBV_QP_RETRY_CNT = 1 << 10,
  IBV_QP_RNR_RETRY = 1 << 11,
  IBV_QP_RQ_PSN = 1 << 12,
  IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13,
  IBV_QP_ALT_PATH = 1 << 14,
  IBV_QP_MIN_RNR_TIMER = 1 << 15,
  IBV_QP_SQ_PSN = 1 << 16,
  IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
  IBV_QP_PATH_MIG_STATE = 1 << 18,
  IBV_QP_CAP = 1 << 19,
  IBV_QP_DEST_QPN = 1 << 20
};

struct ibv_qp {
  struct ibv_context* context;
  void* qp_context;
  struct ibv_pd* pd;
  struct ibv_cq* send_cq;
  struct ibv_cq* recv_cq;
  struct ibv_srq* srq;
  uint32_t handle;
  uint32_t qp_num;
  enum ibv_qp_state state;
  enum ibv_qp_type qp_type;
  pthread_mutex_t mutex;
  pthread_cond_t cond;
  uint32_t events_completed;
};

struct ibv_sge {
  uint64_t addr;
  uint32_t length;
  uint32_t lkey;
};

enum ibv_wr_opcode {
  IBV_WR_RDMA_WRITE = 0,
  IBV_WR_RDMA_WRITE_WITH_IMM = 1,
  IBV_WR_SEND = 2,
  IBV_WR_SEND_WITH_IMM = 3,
  IBV_WR_RDMA_READ = 4,
  IBV_WR_ATOMIC_CMP_AND_SWP = 5,
  IBV_WR_ATOMIC_FETCH_AND_ADD = 6
};
enum ibv_send_flags { IBV_SEND_FENCE = 1, IBV_SEND_SIGNALED = 2, IBV_SEND_SOLICITED = 4, IBV_SEND_INLINE = 8 };

struct ibv_mw_bind_info {
  struct ibv_mr* mr;
  uint64_t addr;
  uint64_t length;
  unsigned int mw_access_flags;
};

struct ibv_send_wr {
  uint64_t wr_id;
  struct ibv_send_wr* next;
  struct ibv_sge* sg_list;
  int num_sge;
  enum ibv_wr_opcode opcode;
  unsigned int send_flags;
  union {
    uint32_t imm_data;  // big endian on the wire
    uint32_t invalidate_rkey;
  };
  union {
    struct {
      uint64_t remote_addr;
      uint32_t rkey;
    } rdma;
    struct {
      uint64_t remote_addr;
      uint64_t compare_add;
      uint64_t swap;
      uint32_t rkey;
    } atomic;
    struct {
      struct ibv_ah* ah;
      uint32_t remote_qpn;
      uint32_t remote_qkey;
    } ud;
  } wr;
  union {
    struct {
      uint32_t remote_srqn;
    } xrc;
  } qp_type;
  union {
    struct {
      struct ibv_mw* mw;
      uint32_t rkey;
      struct ibv_mw_bind_info bind_info;
    } bind_mw;
    struct {
      void* hdr;
      uint16_t hdr_sz;
      uint16_t mss;
    } tso;
  };
};

struct ibv_recv_wr {
  uint64_t wr_id;
  struct ibv_recv_wr* next;
  struct ibv_sge* sg_list;
  int num_sge;
};

enum ibv_wc_status {
  IBV_WC_SUCCESS = 0,
  IBV_WC_LOC_LEN_ERR = 1,
  IBV_WC_LOC_QP_OP_ERR = 2,
  IBV_WC_LOC_EEC_OP_ERR = 3,
  IBV_WC_LOC_PROT_ERR = 4,
  IBV_WC_WR_FLUSH_ERR = 5,
  IBV_WC_MW_BIND_ERR = 6,
  IBV_WC_BAD_RESP_ERR = 7,
  IBV_WC_LOC_ACCESS_ERR = 8,
  IBV_WC_REM_INV_REQ_ERR = 9,
  IBV_WC_REM_ACCESS_ERR = 10,
  IBV_WC_REM_OP_ERR = 11,
  IBV_WC_RETRY_EXC_ERR = 12,
  IBV_WC_RNR_RETRY_EXC_ERR = 13,
  IBV_WC_GENERAL_ERR = 21
};
enum ibv_wc_opcode {
  IBV_WC_SEND = 0,
  IBV_WC_RDMA_WRITE = 1,
  IBV_WC_RDMA_READ = 2,
  IBV_WC_COMP_SWAP = 3,
  IBV_WC_FETCH_ADD = 4,
  IBV_WC_RECV = 1 << 7,
  IBV_WC_RECV_RDMA_WITH_IMM = (1 << 7) + 1
};
enum ibv_wc_flags { IBV_WC_GRH = 1, IBV_WC_WITH_IMM = 2 };

struct ibv_wc {
  uint64_t wr_id;
  enum ibv_wc_status status;
  enum ibv_wc_opcode opcode;
  uint32_t vendor_err;
  uint32_t byte_len;
  union {
    uint32_t imm_data;  // big endian on the wire
    uint32_t invalidated_rkey;
  };
  uint32_t qp_num;
  uint32_t src_qp;
  unsigned int wc_flags;
  uint16_t pkey_index;
  uint16_t slid;
  uint8_t sl;
  uint8_t dlid_path_bits;
};

// The fast-path entry points are not exported symbols of libibverbs: <infiniband/verbs.h> implements ibv_poll_cq,
// ibv_post_send and ibv_post_recv as inline calls through this table of the device context. Slots this library does not
// call are kept as anonymous pointers, in the order of the 1.x ABI.
struct ibv_context_ops {
  void* compat_query_device;
  void* compat_query_port;
  void* compat_alloc_pd;
  void* compat_dealloc_pd;
  void* compat_reg_mr;
  void* compat_rereg_mr;
  void* compat_dereg_mr;
  void* alloc_mw;
  void* bind_mw;
  void* dealloc_mw;
  void* compat_create_cq;
  int (*poll_cq)(struct ibv_cq* cq, int num_entries, struct ibv_wc* wc);
  void* req_notify_cq;
  void* compat_cq_event;
  void* compat_resize_cq;
  void* compat_destroy_cq;
  void* compat_create_srq;
  void* compat_modify_srq;
  void* compat_query_srq;
  void* compat_destroy_srq;
  void* post_srq_recv;
  void* compat_create_qp;
  void* compat_query_qp;
  void* compat_modify_qp;
  void* compat_destroy_qp;
  int (*post_send)(struct ibv_qp* qp, struct ibv_send_wr* wr, struct ibv_send_wr** bad_wr);
  int (*post_recv)(struct ibv_qp* qp, struct ibv_recv_wr* wr, struct ibv_recv_wr** bad_wr);
  void* compat_create_ah;
  void* compat_destroy_ah;
  void* compat_attach_mcast;
  void* compat_detach_mcast;
  void* compat_async_event;
};

struct ibv_context {
  struct ibv_device* device;
  struct ibv_context_ops ops;
  int cmd_fd;
  int async_fd;
  int num_comp_vectors;
  pthread_mutex_t mutex;
  void* abi_compat;
};

}  // extern "C"

#endif  // MSCCLPP_IB_SYSTEM_HEADER
