/* Minimal stand-in for libnuma's <numa.h>, for building the reference on an image without libnuma-dev.
 * Only what the reference's numa.cc uses: the v1 node mask and numa_bind_compat, implemented with the
 * set_mempolicy / sched_setaffinity system calls. */
#ifndef BASELINE_DEPS_NUMA_H_
#define BASELINE_DEPS_NUMA_H_
#ifdef __cplusplus
extern "C" {
#endif
#define NUMA_NUM_NODES 128
typedef struct {
  unsigned long n[NUMA_NUM_NODES / (sizeof(unsigned long) * 8)];
} nodemask_t;
static inline void nodemask_zero(nodemask_t* m) {
  for (unsigned i = 0; i < sizeof(m->n) / sizeof(m->n[0]); ++i) m->n[i] = 0;
}
static inline void nodemask_set_compat(nodemask_t* m, int node) {
  m->n[node / (8 * sizeof(unsigned long))] |= 1UL << (node % (8 * sizeof(unsigned long)));
}
int numa_available(void);
int numa_num_configured_nodes(void);
void numa_bind_compat(nodemask_t* mask);
#ifdef __cplusplus
}
#endif
#endif
