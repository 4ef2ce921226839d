// Interface of the tcgen05 grouped expert kernels (experts_tc.cu).
#pragma once
#include "common.cuh"

namespace nvmoe {

// Shapes the tensor-core path takes: columns in whole 32-blocks with a power-of-two activation
// scale per block (always true for the plan's own quantiser).
bool tc_shape_supported(const nvmoe_geometry& g);
// Whether "automatic" picks the tensor-core path.
bool tc_enabled_by_default();
void tc_configure_kernels();
// Encodes the template tensor map of a [rows][cols] weight matrix (any 32-byte aligned device address
// will do: it is replaced per expert). False when the shape cannot use TMA.
bool tc_encode_weight_map(void* map128, void* any_device_address, uint32_t rows, uint32_t cols);
// The same for a matrix held as one E4M3 byte per element (pre-expanded or native FP8 resources).
bool tc_encode_weight_map_bytes(void* map128, void* any_device_address, uint32_t rows, uint32_t cols);
// Encodes the tensor map of an expert-grouped activation matrix [rows][cols] of E4M3 bytes with a box of
// n_tile rows x 128 bytes (the operand tile of one K block). False when tensor maps are unavailable.
bool tc_encode_activation_map(void* map128, void* base, uint32_t rows, uint32_t cols, uint32_t n_tile);
// per-expert tensor maps = template + the expert's weight address (p.tmaps must be set)
void launch_build_tensormaps_tc(const ExpertLaunch& p, bool gate_up, const uint8_t* templ, cudaStream_t stream);
// token tile size of a stage for this many tokens (the (expert, token tile) list must be built with it)
uint32_t tc_token_tile_for(uint32_t tokens, uint32_t routes_per_token, uint32_t num_experts, bool gate_up);
// which of a stage's four tile sizes (and activation tensor maps) that is
uint32_t tc_token_tile_index(uint32_t n_tile);
// bytes of the derived (tiled) scale copy of one expert matrix with `rows` x `cols` elements
size_t tc_derived_scale_bytes(uint32_t rows, uint32_t cols);
// re-tiles the scales of every expert whose scale record changed since the last call
void launch_derive_scales_tc(const ExpertLaunch& p, bool gate_up, cudaStream_t stream);
void launch_gate_up_tc(const ExpertLaunch& p, cudaStream_t stream);
void launch_down_tc(const ExpertLaunch& p, cudaStream_t stream);

}  // namespace nvmoe
