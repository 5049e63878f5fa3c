#include "nt_core.cuh"
extern "C" {
int nt_comm_unique_id(uint8_t *) { ntb::set_last_error("comm not built"); return NT_ERR_RUNTIME; }
int nt_comm_init(int, int, const uint8_t *) { ntb::set_last_error("comm not built"); return NT_ERR_RUNTIME; }
int nt_comm_allreduce_sum(nt_storage *) { ntb::set_last_error("comm not built"); return NT_ERR_RUNTIME; }
int nt_comm_wait(void) { return NT_OK; }
int nt_comm_destroy(void) { return NT_OK; }
}
