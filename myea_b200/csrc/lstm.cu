// placeholder, replaced below
#include "net.cuh"
namespace myea {
int lstm_create(myea_b200_net *, LayerPlan &) { return MYEA_E_UNSUPPORTED; }
void lstm_destroy(LayerPlan &) {}
int lstm_forward(myea_b200_net *, LayerPlan &, const float *, long long) { return MYEA_E_UNSUPPORTED; }
int lstm_backward(myea_b200_net *, LayerPlan &) { return MYEA_E_UNSUPPORTED; }
int lstm_backward_to_input(myea_b200_net *, LayerPlan &, float *, const LayerPlan &) { return MYEA_E_UNSUPPORTED; }
int lstm_update_derivative_weight(myea_b200_net *, LayerPlan &, const float *, long long) { return MYEA_E_UNSUPPORTED; }
int lstm_set_zoneout(myea_b200_net *, LayerPlan &, const uint8_t *, const uint8_t *, uint64_t) { return MYEA_E_UNSUPPORTED; }
float *lstm_output_errors(LayerPlan &) { return nullptr; }
}
