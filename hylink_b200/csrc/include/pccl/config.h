/* PCCL-compatible configuration record (pcie-ccl-cuda/include/pccl/config.h:
 * 10-20). Every field can also be set through the environment; a zero / NULL
 * field means "use the environment or the default". */
#ifndef PCCL_CONFIG_H
#define PCCL_CONFIG_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int nranks;
  int device_count;
  const int* gpu_ids;
  const char* bootstrap_addr;   /* single node only: must be NULL */
  size_t host_buffer_size;      /* bytes of pinned staging per NUMA node */
  const char* gpu_numa_map;     /* "00001111" or "0,0,0,0,1,1,1,1" */
  const char* ir_path;          /* directory (or one file) of schedule XML */
} pcclConfig_t;

#define PCCL_CONFIG_DEFAULT { 0, 0, NULL, NULL, 0, NULL, NULL }

/* Applies the non-zero fields process-wide (must precede pcclCommInitRank). */
int pcclSetConfig(const pcclConfig_t* config);

#ifdef __cplusplus
}
#endif
#endif /* PCCL_CONFIG_H */
