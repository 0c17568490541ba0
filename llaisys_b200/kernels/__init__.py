"""Python faces of the CUDA kernels under `csrc/`.  Every function takes torch tensors on the
CUDA device, launches on torch's current stream and raises if the launch is refused.  There is
no CPU path: without a device, or without a compiler for the kernels, these functions fail."""
from . import heads, mixers, ops
from .heads import branch_mean, diff_combine, head_prep, pool_append, scale_, stream_join
from .mixers import mingru, head_gate_, rope_pairs_, gla_out, gla_scan, head_matmul, latent_append, latent_attention, latent_prep, require_latent_row
from .ops import (act_rows_, stream_update, glu, scaled_norm_add, DT, AttnExtras, KernelError, embedding_pair, moe_combine, moe_gather_rows, moe_gemm, moe_gemm_tc, moe_plan, moe_route, moe_tc_ok, moe_tc_tile_rows, relu_squared_, rmsnorm_multi, rope_lead_append, add_rmsnorm, decode_clusters16, decode_fusion_ok, dense_binary, argmax, attention_decode, attention_prefill,
                  embedding, fill_normal, gather_i32, into_plan, launch_count, linear, linear_into, linear_into_ok, linear_swiglu, mlp_fused, mlp_fused_ok, prefill_tc_ok, require_head_dim, residual_add, rope_append, sample, scatter_i32, swiglu, tc_error, tc_plan, uniform)

__all__ = ["branch_mean", "diff_combine", "head_prep", "pool_append", "scale_", "stream_join", "act_rows_", "stream_update", "mingru", "head_gate_", "rope_pairs_", "gla_out", "gla_scan", "head_matmul", "latent_append", "latent_attention", "latent_prep", "require_latent_row", "glu", "scaled_norm_add", "DT", "AttnExtras", "KernelError", "embedding_pair", "moe_combine", "moe_gather_rows", "moe_gemm", "moe_gemm_tc", "moe_plan", "moe_route", "moe_tc_ok", "moe_tc_tile_rows", "relu_squared_", "rmsnorm_multi", "rope_lead_append", "add_rmsnorm", "decode_clusters16", "decode_fusion_ok", "dense_binary", "argmax", "attention_decode", "attention_prefill",
           "embedding", "fill_normal", "gather_i32", "into_plan", "launch_count", "linear", "linear_into", "linear_into_ok", "linear_swiglu", "mlp_fused", "mlp_fused_ok", "prefill_tc_ok", "require_head_dim", "residual_add", "rope_append", "sample", "scatter_i32", "swiglu", "tc_error", "tc_plan", "uniform"]
