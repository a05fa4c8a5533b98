"""ctypes declarations of the parts of include/cogito.h that the CPU tests exercise."""
from __future__ import annotations

import ctypes
import sys
from ctypes import (CFUNCTYPE, POINTER, Structure, c_bool, c_char, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint, c_uint8, c_uint16, c_uint32, c_uint64, c_void_p)
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "bindings"))
import cogito as cg  # noqa: E402

TensorP = cg.TensorP
FP = POINTER(c_float)
IP = POINTER(c_int)


class Layer(Structure):
    pass


LayerP = POINTER(Layer)
Layer._fields_ = [("name", c_char_p), ("weights", TensorP), ("bias", TensorP), ("input", TensorP), ("output", TensorP),
                  ("forward", CFUNCTYPE(TensorP, LayerP, TensorP)), ("backward", CFUNCTYPE(None, LayerP, TensorP)),
                  ("free", CFUNCTYPE(None, LayerP)), ("num_params", CFUNCTYPE(c_int, LayerP)),
                  ("get_params", CFUNCTYPE(POINTER(TensorP), LayerP))]


class Optimizer(Structure):
    _fields_ = [("learning_rate", c_float), ("params", POINTER(TensorP)), ("num_params", c_int), ("t", c_int),
                ("use_mixed_precision", c_bool), ("loss_scale", c_float), ("scale_window", c_int), ("scale_factor", c_float),
                ("scale_backoff", c_int), ("use_master_weights", c_bool), ("master_params", POINTER(TensorP)),
                ("max_grad_norm", c_float), ("step", c_void_p), ("zero_grad", c_void_p), ("free", c_void_p)]


class TensorQuant(Structure):
    _fields_ = [("data", POINTER(c_uint8)), ("scales", FP), ("zeros", FP), ("shape", IP), ("ndim", c_int), ("size", c_int),
                ("quant_type", c_int), ("group_size", c_int), ("num_groups", c_int), ("symmetric", c_bool)]


class KVCache(Structure):
    _fields_ = [("k_cache", POINTER(c_uint8)), ("v_cache", POINTER(c_uint8)), ("k_scales", FP), ("v_scales", FP),
                ("current_len", c_int), ("max_seq_len", c_int), ("num_layers", c_int), ("n_heads", c_int),
                ("head_dim", c_int), ("group_size", c_int)]


class FlashConfig(Structure):
    _fields_ = [("block_m", c_int), ("block_n", c_int), ("num_warps", c_int), ("num_stages", c_int),
                ("use_register_tiling", c_bool), ("split_k", c_int), ("use_persistent", c_bool), ("sm_count", c_int)]


class FlashParams(Structure):
    _fields_ = [("Q", TensorP), ("K", TensorP), ("V", TensorP), ("O", TensorP), ("dO", TensorP), ("dQ", TensorP),
                ("dK", TensorP), ("dV", TensorP), ("L", TensorP), ("mask", TensorP),
                ("batch_size", c_int), ("seqlen_q", c_int), ("seqlen_k", c_int), ("n_heads", c_int), ("n_kv_heads", c_int),
                ("d_head", c_int), ("softmax_scale", c_float), ("dropout_prob", c_float), ("mask_type", c_int),
                ("window_size", c_int), ("alibi_slopes", FP), ("config", FlashConfig), ("is_training", c_bool), ("softmax_lse", FP),
                ("dropout_mask", FP), ("operand_mode", c_uint)]


class TransformerConfig(Structure):
    _fields_ = [("hidden_size", c_int), ("num_heads", c_int), ("num_kv_heads", c_int), ("head_dim", c_int),
                ("intermediate_size", c_int), ("norm_eps", c_float), ("dropout_prob", c_float), ("use_bias", c_bool),
                ("pre_norm", c_bool), ("use_rms_norm", c_bool), ("use_swiglu", c_bool)]


class ScheduleStep(Structure):
    _fields_ = [("action", c_int), ("microbatch_id", c_int), ("stage_id", c_int)]


class Pipeline(Structure):
    _fields_ = [("num_stages", c_int), ("micro_batch_size", c_int), ("num_microbatches", c_int), ("global_batch_size", c_int),
                ("stages", c_void_p), ("schedule", POINTER(ScheduleStep)), ("schedule_len", c_int), ("pp_group", c_void_p),
                ("dp_group", c_void_p), ("use_recompute", c_bool), ("activation_cache", c_void_p), ("last_loss", c_float),
                ("impl", c_void_p)]


class Group(Structure):
    _fields_ = [("mode", c_int), ("world_size", c_int), ("rank", c_int), ("ranks", IP), ("comm", c_void_p), ("stream", c_void_p)]


class Parallel3D(Structure):
    _fields_ = [("dp_size", c_int), ("tp_size", c_int), ("pp_size", c_int), ("dp_rank", c_int), ("tp_rank", c_int),
                ("pp_rank", c_int), ("world_size", c_int), ("world_rank", c_int), ("dp_group", POINTER(Group)),
                ("tp_group", POINTER(Group)), ("pp_group", POINTER(Group))]


class TokenTree(Structure):
    _fields_ = [("tokens", IP), ("probs", POINTER(FP)), ("parents", IP), ("depth", c_int), ("num_tokens", c_int),
                ("capacity", c_int), ("vocab_size", c_int)]


LogitsFn = CFUNCTYPE(None, c_void_p, IP, c_int, c_int, FP)


class SpecDecoder(Structure):
    _fields_ = [("draft_model", c_void_p), ("target_model", c_void_p), ("gamma", c_int), ("temperature", c_float),
                ("top_p", c_float), ("top_k", c_int), ("total_draft_tokens", c_int), ("accepted_draft_tokens", c_int),
                ("num_steps", c_int), ("avg_acceptance_rate", c_float), ("draft_fn", LogitsFn), ("target_fn", LogitsFn),
                ("vocab_size", c_int), ("rng_state", c_uint)]


class MemoryStats(Structure):
    _fields_ = [("total_allocated", c_size_t), ("total_cached", c_size_t), ("peak_allocated", c_size_t), ("num_allocs", c_int),
                ("num_frees", c_int), ("cache_hits", c_int), ("cache_misses", c_int), ("buddy_splits", c_int),
                ("buddy_coalesces", c_int), ("fragmentation", c_float), ("total_in_use", c_size_t), ("peak_usage", c_size_t),
                ("cache_hit_rate", c_size_t), ("num_bins_used", c_int)]


class IrNode(Structure):
    pass


IrNode._fields_ = [("opcode", c_int), ("id", c_int), ("input_ids", IP), ("num_inputs", c_int), ("output_id", c_int),
                   ("output_shape", c_int * 8), ("output_ndim", c_int), ("attributes", c_void_p), ("attr_size", c_size_t),
                   ("schedule_order", c_int), ("can_fuse", c_bool), ("fusion_type", c_int), ("fused_with", POINTER(IrNode)),
                   ("dead", c_bool)]


class IrGraph(Structure):
    _fields_ = [("nodes", POINTER(POINTER(IrNode))), ("num_nodes", c_int), ("capacity", c_int), ("tensors", POINTER(TensorP)),
                ("num_tensors", c_int), ("tensor_capacity", c_int), ("input_node_ids", IP), ("num_inputs", c_int),
                ("output_node_ids", IP), ("num_outputs", c_int), ("opt_level", c_int)]


class JitCompiler(Structure):
    _fields_ = [("graph", POINTER(IrGraph)), ("backend", c_int), ("source_code", c_char_p), ("source_len", c_size_t),
                ("compiled_module", c_void_p), ("compiled_kernel", c_void_p), ("is_compiled", c_bool),
                ("shared_memory_bytes", c_int), ("registers_per_thread", c_int), ("occupancy", c_int),
                ("shape_hash", c_uint64), ("pattern_hash", c_uint64)]


class FusionGroup(Structure):
    _fields_ = [("nodes", POINTER(POINTER(IrNode))), ("num_nodes", c_int), ("capacity", c_int), ("fusion_type", c_int),
                ("kernel_name", c_char_p), ("kernel_code", c_char_p), ("output_shape", IP), ("output_ndim", c_int),
                ("memory_saved", c_size_t), ("flops", c_size_t), ("arithmetic_intensity", c_float),
                ("schedule_priority", c_int), ("is_valid", c_bool)]


class FusionPass(Structure):
    _fields_ = [("graph", POINTER(IrGraph)), ("groups", POINTER(POINTER(FusionGroup))), ("num_groups", c_int),
                ("max_groups", c_int), ("max_fusion_depth", c_int), ("enable_epilogue", c_bool), ("enable_attention", c_bool),
                ("aggressive", c_bool)]


class MixedPrecision(Structure):
    _fields_ = [("params", POINTER(TensorP)), ("model_params", c_void_p), ("num_params", c_int), ("loss_scale", c_float),
                ("min_loss_scale", c_float), ("max_loss_scale", c_float), ("scale_factor", c_float), ("scale_window", c_int),
                ("steps_since_overflow", c_int), ("found_overflow", c_bool), ("max_grad_norm", c_float),
                ("learning_rate", c_float), ("num_skipped", c_int), ("num_steps", c_int)]


_DECLARED = False


def L():
    """The library with argument / result types set for everything the tests call."""
    global _DECLARED
    lib = cg.lib()
    if _DECLARED:
        return lib
    P, V, I, F, B, SZ = c_void_p, None, c_int, c_float, c_bool, c_size_t
    table = {
        # layers / model
        "cg_linear_new": (LayerP, I, I, B), "cg_relu_new": (LayerP,), "cg_sigmoid_new": (LayerP,), "cg_tanh_new": (LayerP,),
        "cg_softmax_new": (LayerP,), "cg_dropout_new": (LayerP, F), "cg_dropout_set_training": (V, LayerP, B),
        "cg_batchnorm_new": (LayerP, I, F, F), "cg_batchnorm_set_training": (V, LayerP, B), "cg_rmsnorm_new": (LayerP, I, F),
        "cg_swiglu_new": (LayerP,), "cg_conv2d_new": (LayerP, I, I, I, I, I, B), "cg_maxpool2d_new": (LayerP, I, I),
        "cg_flatten_new": (LayerP,), "cg_layer_free": (V, LayerP), "cg_sequential_new": (LayerP,),
        "cg_sequential_add": (V, LayerP, LayerP), "cg_sequential_forward": (TensorP, LayerP, TensorP),
        "cg_sequential_backward": (V, LayerP, TensorP), "cg_sequential_free": (V, LayerP),
        "cg_sequential_zero_grad": (V, LayerP), "cg_sequential_num_params": (I, LayerP),
        "cg_sequential_get_params": (POINTER(TensorP), LayerP),
        "cg_transformer_block_new": (LayerP, TransformerConfig), "cg_transformer_forward": (TensorP, LayerP, TensorP, TensorP),
        # losses / optimizers
        "cg_mse_loss": (TensorP, TensorP, TensorP, I), "cg_cross_entropy_loss": (TensorP, TensorP, TensorP, B, I),
        "cg_softmax_cross_entropy_loss": (TensorP, TensorP, TensorP, I), "cg_bce_loss": (TensorP, TensorP, TensorP, I),
        "cg_bce_with_logits_loss": (TensorP, TensorP, TensorP, I), "cg_l1_loss": (TensorP, TensorP, TensorP, I),
        "cg_smooth_l1_loss": (TensorP, TensorP, TensorP, F, I),
        "cg_sgd_new": (POINTER(Optimizer), POINTER(TensorP), I, F, F, F, B),
        "cg_adam_new": (POINTER(Optimizer), POINTER(TensorP), I, F, F, F, F, F),
        "cg_sgd_new_for_sequential": (POINTER(Optimizer), LayerP, F, F, F, B),
        "cg_adam_new_for_sequential": (POINTER(Optimizer), LayerP, F, F, F, F, F),
        "cg_optimizer_step": (V, POINTER(Optimizer)), "cg_optimizer_zero_grad": (V, POINTER(Optimizer)),
        "cg_optimizer_free": (V, POINTER(Optimizer)), "cg_optimizer_step_lr": (V, POINTER(Optimizer), I, I, F),
        "cg_optimizer_exp_lr": (V, POINTER(Optimizer), F, F),
        "cg_optimizer_enable_loss_scaling": (V, POINTER(Optimizer), F, F, I),
        "cg_optimizer_enable_master_weights": (V, POINTER(Optimizer)), "cg_optimizer_update_scale": (B, POINTER(Optimizer), F),
        # tensor helpers
        "cg_tensor_add": (V, TensorP, TensorP, TensorP), "cg_tensor_mul": (V, TensorP, TensorP, TensorP),
        "cg_tensor_matmul": (V, TensorP, TensorP, TensorP), "cg_tensor_sum": (V, TensorP, I, TensorP),
        "cg_tensor_exp": (V, TensorP, TensorP), "cg_tensor_transpose": (V, TensorP, TensorP),
        "cg_tensor_add_broadcast": (TensorP, TensorP, TensorP), "cg_tensor_cat": (TensorP, POINTER(TensorP), I, I),
        "cg_tensor_stack": (TensorP, POINTER(TensorP), I), "cg_tensor_clone": (TensorP, TensorP),
        "cg_grad_check": (B, CFUNCTYPE(None, TensorP, TensorP), TensorP, TensorP, F, F),
        "cg_arena_new": (P, SZ), "cg_arena_alloc": (P, P, SZ, SZ), "cg_arena_clear": (V, P), "cg_arena_free": (V, P),
        "cg_arena_total_used": (SZ, P), "cg_tensor_zeros_arena": (TensorP, P, IP, I, B),
        # data / io
        "cg_save_model": (V, c_char_p, POINTER(TensorP), POINTER(c_char_p), I),
        "cg_load_model": (V, c_char_p, POINTER(POINTER(TensorP)), POINTER(POINTER(c_char_p)), IP),
        "cg_mnist_load": (P, c_char_p, c_char_p), "cg_mnist_free": (V, P),
        "cg_data_iter_new": (P, TensorP, TensorP, I, B, c_uint), "cg_data_iter_next": (B, P, POINTER(TensorP), POINTER(TensorP)),
        "cg_data_iter_free": (V, P), "cg_dataloader_new": (P, TensorP, TensorP, I, B, c_uint),
        "cg_dataloader_next": (B, P, POINTER(TensorP), POINTER(TensorP), IP), "cg_dataloader_num_batches": (I, P),
        "cg_dataloader_reset": (V, P), "cg_dataloader_free": (V, P), "cg_tensor_onehot": (TensorP, TensorP, I),
        "cg_compute_accuracy": (F, TensorP, TensorP, I),
        "cg_profiler_init": (V,), "cg_profiler_begin_layer": (V, c_char_p), "cg_profiler_end_layer": (V, c_char_p),
        "cg_profiler_count": (I, c_char_p), "cg_profiler_total_ms": (ctypes.c_double, c_char_p), "cg_profiler_reset": (V,),
        "cg_fp32_to_bf16": (c_uint16, F), "cg_bf16_to_fp32": (F, c_uint16),
        "cg_mixed_precision_new": (POINTER(MixedPrecision), POINTER(TensorP), I), "cg_mp_backward": (B, POINTER(MixedPrecision), P),
        "cg_mp_step": (V, POINTER(MixedPrecision)), "cg_mixed_precision_free": (V, POINTER(MixedPrecision)),
        # quant
        "cg_quantize_int4": (POINTER(TensorQuant), TensorP, I), "cg_quantize_nf4": (POINTER(TensorQuant), TensorP, I),
        "cg_quantize_gptq": (POINTER(TensorQuant), TensorP, TensorP, I, I), "cg_quantize_awq": (POINTER(TensorQuant), TensorP, TensorP, I),
        "cg_dequantize": (TensorP, POINTER(TensorQuant)), "cg_tensor_quant_free": (V, POINTER(TensorQuant)),
        "cg_matmul_int4": (V, TensorP, POINTER(TensorQuant), TensorP), "cg_gemv_int4": (V, TensorP, POINTER(TensorQuant), TensorP),
        "cg_kv_cache_int4_new": (POINTER(KVCache), I, I, I, I, I), "cg_kv_cache_int4_append": (V, POINTER(KVCache), I, TensorP, TensorP),
        "cg_kv_cache_int4_get": (V, POINTER(KVCache), I, TensorP, TensorP), "cg_kv_cache_int4_free": (V, POINTER(KVCache)),
        "cg_kv_cache_int4_truncate": (V, POINTER(KVCache), I), "cg_attention_int4_kv": (V, TensorP, POINTER(KVCache), I, TensorP),
        "cg_calibration_new": (P, I), "cg_calibration_update": (V, P, TensorP), "cg_calibration_compute_scales": (V, P, FP, FP, I),
        "cg_calibration_free": (V, P),
        # attention
        "cg_flash_attn_params_new": (POINTER(FlashParams), TensorP, TensorP, TensorP, I, F),
        "cg_flash_attention_forward_cpu": (V, POINTER(FlashParams)), "cg_flash_attention_backward_cpu": (V, POINTER(FlashParams)),
        "cg_flash_attn_params_free": (V, POINTER(FlashParams)), "cg_apply_rope": (V, FP, FP, I, I, I, I, F),
        "cg_alibi_slopes": (V, FP, I), "cg_flash_attn_autotune": (FlashConfig, I, I, I, I),
        # inference
        "cg_sample_seed": (V, c_uint), "cg_sample_temperature": (I, FP, I, F), "cg_sample_top_p": (I, FP, I, F),
        "cg_sample_top_k": (I, FP, I, I), "cg_sample_typical": (I, FP, I, F), "cg_acceptance_prob": (F, F, F),
        "cg_sample_corrected": (I, FP, FP, I),
        "cg_speculative_decoder_new": (POINTER(SpecDecoder), P, P, I), "cg_speculative_set_models": (V, POINTER(SpecDecoder), LogitsFn, LogitsFn, I),
        "cg_speculative_generate": (TensorP, POINTER(SpecDecoder), TensorP, I, F, F), "cg_speculative_decoder_free": (V, POINTER(SpecDecoder)),
        "cg_token_tree_new": (POINTER(TokenTree), I), "cg_token_tree_add_token": (V, POINTER(TokenTree), I, FP),
        "cg_token_tree_add_child": (I, POINTER(TokenTree), I, I, FP), "cg_token_tree_free": (V, POINTER(TokenTree)),
        "cg_tree_attention_mask": (TensorP, POINTER(TokenTree), I),
        "cg_eagle_draft_new": (P, P), "cg_eagle_generate_tree": (POINTER(TokenTree), P, TensorP, I), "cg_eagle_draft_free": (V, P),
        # pipeline
        "cg_pipeline_gen_1f1b_stage": (POINTER(ScheduleStep), I, I, I, IP), "cg_pipeline_gen_interleaved_stage": (POINTER(ScheduleStep), I, I, I, I, IP),
        "cg_pipeline_new": (POINTER(Pipeline), I, I), "cg_pipeline_set_stage": (V, POINTER(Pipeline), I, P, I),
        "cg_pipeline_forward_backward": (V, POINTER(Pipeline), TensorP, TensorP), "cg_pipeline_free": (V, POINTER(Pipeline)),
        "cg_3d_parallel_new": (POINTER(Parallel3D), I, I, I), "cg_3d_parallel_init_from_world": (V, POINTER(Parallel3D), I, I),
        "cg_3d_parallel_free": (V, POINTER(Parallel3D)),
        # memory
        "cg_memory_pool_new": (P,), "cg_pool_alloc": (P, P, SZ), "cg_pool_free": (V, P, P), "cg_memory_pool_free": (V, P),
        "cg_subbin_index": (I, SZ), "cg_memory_fragmentation": (F, P), "cg_pool_trim": (V, P),
        "cg_buddy_new": (P, P, SZ), "cg_buddy_alloc": (P, P, SZ), "cg_buddy_free": (V, P, P, SZ), "cg_buddy_destroy": (V, P),
        "cg_buddy_splits": (I, P), "cg_buddy_coalesces": (I, P),
        "cg_memory_planner_new": (P,), "cg_memory_plan_analyze": (V, P, P), "cg_memory_plan_bytes": (SZ, P),
        "cg_can_reuse_memory": (B, P, I, I), "cg_planned_alloc": (P, P, SZ, I), "cg_planned_free": (V, P, P, I),
        "cg_memory_planner_free": (V, P), "cg_cuda_graph_capture_begin": (V, P), "cg_cuda_graph_capture_end": (V, P),
        "cg_cuda_graph_replay": (V, P), "cg_cuda_graph_needs_update": (B, P), "cg_memory_get_stats": (MemoryStats, P),
        # symbolic
        "cg_dim_const": (P, c_int64), "cg_dim_var": (P, c_char_p), "cg_dim_inferred": (P, P), "cg_dim_constrain": (V, P, c_int64, c_int64),
        "cg_expr_var": (P, c_char_p), "cg_expr_const": (P, c_int64), "cg_expr_mul": (P, P, P), "cg_expr_add": (P, P, P),
        "cg_expr_floordiv": (P, P, P), "cg_expr_to_string": (P, P), "cg_expr_free": (V, P),
        "cg_shape_new": (P, POINTER(P), I), "cg_shape_from_ints": (P, IP, I), "cg_shape_matmul": (P, P, P), "cg_shape_broadcast": (P, P, P),
        "cg_shape_is_dynamic": (B, P), "cg_shape_resolve": (B, P, POINTER(c_int64), POINTER(c_char_p), I, IP), "cg_shape_free": (V, P),
        "cg_shape_hash": (c_uint64, P), "cg_shape_specialize": (P, P, POINTER(c_int64), POINTER(c_char_p), I),
        "cg_shape_guards_hold": (B, P, POINTER(c_int64), POINTER(c_char_p), I), "cg_shape_specialization_free": (V, P),
        # jit
        "cg_jit_begin_trace": (V,), "cg_jit_end_trace": (POINTER(IrGraph),), "cg_ir_graph_new": (POINTER(IrGraph),),
        "cg_ir_graph_free": (V, POINTER(IrGraph)), "cg_ir_graph_tensor_id": (I, POINTER(IrGraph), TensorP),
        "cg_ir_graph_add_node": (POINTER(IrNode), POINTER(IrGraph), I, IP, I, I, P, SZ), "cg_ir_graph_mark_output": (V, POINTER(IrGraph), TensorP),
        "cg_ir_graph_live_nodes": (I, POINTER(IrGraph)), "cg_ir_optimize": (V, POINTER(IrGraph), I), "cg_ir_cse": (V, POINTER(IrGraph)),
        "cg_ir_dce": (V, POINTER(IrGraph)), "cg_ir_execute": (B, POINTER(IrGraph)),
        "cg_jit_codegen_c": (P, POINTER(IrGraph)), "cg_jit_codegen_cuda": (P, POINTER(IrGraph)),
        "cg_jit_compiler_new": (POINTER(JitCompiler), POINTER(IrGraph), I), "cg_jit_compile": (B, POINTER(JitCompiler)),
        "cg_jit_run": (B, POINTER(JitCompiler)), "cg_jit_compiler_free": (V, POINTER(JitCompiler)),
        "cg_fusion_pass_new": (POINTER(FusionPass), POINTER(IrGraph)), "cg_fusion_analyze": (V, POINTER(FusionPass)),
        "cg_fusion_apply": (V, POINTER(FusionPass)), "cg_fusion_pass_free": (V, POINTER(FusionPass)),
        "cg_fusion_generate_kernel": (P, POINTER(FusionGroup)),
    }
    for name, sig in table.items():
        fn = getattr(lib, name)
        fn.restype = sig[0]
        fn.argtypes = list(sig[1:])
    _DECLARED = True
    return lib


def T(a, requires_grad=False):
    return cg.Tensor.from_numpy(np.asarray(a, dtype=np.float32), requires_grad)


def borrowed(ptr):
    """numpy copy of a tensor the library still owns."""
    c = ptr.contents
    shape = tuple(c.shape[i] for i in range(c.ndim))
    return np.ctypeslib.as_array(c.data, shape=(c.size,)).reshape(shape).copy()


def grad_of(ptr):
    c = ptr.contents
    shape = tuple(c.shape[i] for i in range(c.ndim))
    return np.ctypeslib.as_array(c.grad, shape=(c.size,)).reshape(shape).copy()


def take_string(p):
    """Copy a malloc'd C string and free it."""
    s = ctypes.string_at(p).decode()
    ctypes.CDLL(None).free(ctypes.c_void_p(p))
    return s
