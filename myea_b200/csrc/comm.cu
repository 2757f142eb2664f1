// placeholder, replaced below
#include "net.cuh"
namespace myea {
int comm_all_reduce_sum(myea_b200_net *, float *, size_t) { return MYEA_E_UNSUPPORTED; }
int comm_all_reduce_sum_f64(myea_b200_net *, double *, size_t) { return MYEA_E_UNSUPPORTED; }
void comm_destroy(myea_b200_net *) {}
}
extern "C" int myea_b200_comm_unique_id(uint8_t *) { return MYEA_E_UNSUPPORTED; }
extern "C" int myea_b200_comm_init(myea_handle, int, int, const uint8_t *) { return MYEA_E_UNSUPPORTED; }
