#include "tables.hpp"
#include "layers.hpp"

namespace nve_b200 {

std::shared_ptr<Table> make_gpu_table(const nve_gpu_table_config_t&, nve_key_type_t) {
  throw NotImplemented("GPU cache table: not built yet");
}
std::shared_ptr<EmbeddingLayer> make_linear_uvm_layer(const nve_linear_uvm_layer_config_t&,
                                                      nve_key_type_t, std::shared_ptr<Table>) {
  throw NotImplemented("Linear UVM layer: not built yet");
}

}  // namespace nve_b200
