/* Stand-in libnuma: counts nodes from sysfs, binds memory policy and CPU affinity to the nodes of a mask. */
#define _GNU_SOURCE
#include "numa.h"

#include <dirent.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/syscall.h>
#include <unistd.h>

#define MPOL_BIND 2

int numa_available(void) { return 0; }

int numa_num_configured_nodes(void) {
  DIR* d = opendir("/sys/devices/system/node");
  if (!d) return 1;
  int count = 0;
  struct dirent* e;
  while ((e = readdir(d)) != NULL) {
    if (strncmp(e->d_name, "node", 4) == 0 && e->d_name[4] >= '0' && e->d_name[4] <= '9') ++count;
  }
  closedir(d);
  return count > 0 ? count : 1;
}

static void add_node_cpus(int node, cpu_set_t* set) {
  char path[128];
  snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", node);
  FILE* f = fopen(path, "r");
  if (!f) return;
  char buf[4096];
  if (fgets(buf, sizeof(buf), f)) {
    char* p = buf;
    while (*p && *p != '\n') {
      long a = strtol(p, &p, 10), b = a;
      if (*p == '-') b = strtol(p + 1, &p, 10);
      for (long c = a; c <= b && c < CPU_SETSIZE; ++c) CPU_SET((int)c, set);
      if (*p == ',') ++p;
    }
  }
  fclose(f);
}

void numa_bind_compat(nodemask_t* mask) {
  cpu_set_t set;
  CPU_ZERO(&set);
  for (int node = 0; node < NUMA_NUM_NODES; ++node) {
    if (mask->n[node / (8 * sizeof(unsigned long))] & (1UL << (node % (8 * sizeof(unsigned long))))) add_node_cpus(node, &set);
  }
  if (CPU_COUNT(&set) > 0) sched_setaffinity(0, sizeof(set), &set);
  /* best effort, like libnuma in a container without CAP_SYS_NICE */
  syscall(SYS_set_mempolicy, MPOL_BIND, mask->n, (unsigned long)NUMA_NUM_NODES + 1);
}
