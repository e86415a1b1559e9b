"""Model conversion: weight surgery -> low-bit linear replacement -> forward replacement.

Counterpart of python/llm/src/ipex_llm/transformers/convert.py of the reference
(``is_linear_module`` :138-232, ``_replace_with_low_bit_linear`` :469-748, ``_optimize_pre`` :886-1076,
``ggml_convert_low_bit`` :1079-1171, ``convert_forward`` / ``replace_func`` :1185-1207, ``_optimize_post``
:1253-2042, GPTQ/AWQ repack :379-453).

Design differences from the reference:
* one registry keyed by ``config.model_type`` (``FAMILIES``) instead of a 700-line if/elif chain; families
  that share the transformers-5 attention contract reuse ``models.decoder.decoder_attention_forward``;
* fused 3-D expert parameters (transformers-5 ``MixtralExperts`` & co) become ``LowBitExperts`` so that
  MoE weights are quantized too (the reference's ``nn.Linear`` walk would skip them);
* quantization runs on the GPU when the target device is CUDA.
"""
from __future__ import annotations

import logging
import os
import types
import warnings

import torch
from torch import nn

from ..ops.linear import (BF16Linear, FP16Linear, LowBitLinear, vLLMBF16Linear, vLLMFP16Linear,
                          vLLMLowBitLinear)
from ..ops.embedding import CPUEmbedding, DiskEmbedding, LowBitEmbedding
from ..ops.moe import LowBitExperts, convert_fused_experts, is_fused_experts
from ..quant import qtypes as qt
from ..quant.params import FP4Params, get_block_size
from ..quant.policy import get_cur_qtype_and_imatrix

logger = logging.getLogger(__name__)

_IS_VLLM_AVAILABLE = None


def is_vllm_available():
    global _IS_VLLM_AVAILABLE
    if os.environ.get("IPEX_LLM_NOT_USE_VLLM", None) is not None:
        _IS_VLLM_AVAILABLE = False
    if _IS_VLLM_AVAILABLE is None:
        import importlib.util
        _IS_VLLM_AVAILABLE = importlib.util.find_spec("vllm") is not None and \
            os.environ.get("IPEX_LLM_USE_VLLM", "0") == "1"
    return _IS_VLLM_AVAILABLE


def is_auto_gptq_available():
    import importlib.util
    return importlib.util.find_spec("auto_gptq") is not None


def is_auto_awq_available():
    import importlib.util
    return importlib.util.find_spec("awq") is not None


def is_lm_head(name, model_config, out_features):
    """The vocabulary projection of a generative model (reference convert.py:234-240): only its last position is needed
    during generation.  A masked-LM decoder has the same shape but every position of its output is used."""
    archs = getattr(model_config, "architectures", None) or []
    if any(a.endswith("ForMaskedLM") or a.endswith("ForPreTraining") for a in archs):
        return False
    if name == "lm_head" or getattr(model_config, "vocab_size", None) == out_features:
        return True
    return False


def is_gptq_linear(module):
    return module.__class__.__name__ in ("QuantLinearCudaOld", "QuantLinear") and hasattr(module, "qzeros")


def is_linear_module(module):
    """Recognise every module type that is a plain affine map.  Returns
    ``(is_linear, (in_features, out_features, mp_group))`` (reference convert.py:138-232)."""
    in_features = out_features = mp_group = None
    result = True
    from ..transformers.awq.linear import WQLinear_GEMM
    from ..parallel.tp import ColumnParallelLinear, RowParallelLinear
    if isinstance(module, (LowBitLinear, FP16Linear, BF16Linear)):
        return False, (None, None, None)
    if isinstance(module, nn.Linear):
        in_features, out_features = module.in_features, module.out_features
        mp_group = getattr(module, "mp_group", None)
    elif is_gptq_linear(module):
        in_features, out_features = module.infeatures, module.outfeatures
    elif isinstance(module, WQLinear_GEMM):
        in_features, out_features = module.in_features, module.out_features
    elif isinstance(module, (ColumnParallelLinear, RowParallelLinear)):
        in_features, out_features = module.in_features, module.out_features
        mp_group = module.mp_group if isinstance(module, RowParallelLinear) else None
    elif module.__class__.__name__ == "Conv1D" and hasattr(module, "nf") and module.weight.dim() == 2:
        # GPT-2 style "Conv1D": y = x @ W + b with W stored [in, out]; converted through its transpose
        in_features, out_features = module.weight.shape[0], module.weight.shape[1]
    elif module.__class__.__name__ in ("LinearLayer", "LinearAllreduce"):
        # DeepSpeed AutoTP containers: weight [out, in]; LinearAllreduce carries the process group
        in_features, out_features = module.weight.shape[1], module.weight.shape[0]
        mp_group = getattr(module, "mp_group", None) if module.__class__.__name__ == "LinearAllreduce" else None
    elif module.__class__.__name__ in ("RowParallelLinear", "ColumnParallelLinear", "QKVParallelLinear",
                                       "MergedColumnParallelLinear", "ParallelLMHead", "ReplicatedLinear"):
        # vLLM layers
        in_features = getattr(module, "input_size", None)
        out_features = getattr(module, "output_size", None)
        tp = getattr(module, "tp_size", 1)
        if module.__class__.__name__ == "RowParallelLinear":
            in_features = module.input_size_per_partition
            if tp >= 2:
                from vllm.distributed import get_tensor_model_parallel_group
                mp_group = get_tensor_model_parallel_group()
        elif hasattr(module, "output_size_per_partition"):
            out_features = module.output_size_per_partition
        if module.__class__.__name__ == "ParallelLMHead":
            in_features, out_features = module.embedding_dim, module.num_embeddings_per_partition
    else:
        result = False
    return result, (in_features, out_features, mp_group)


_VLLM_LINEARS = ("RowParallelLinear", "ColumnParallelLinear", "QKVParallelLinear", "MergedColumnParallelLinear",
                 "ReplicatedLinear")


def _is_vllm_linear(module) -> bool:
    return type(module).__name__ in _VLLM_LINEARS and type(module).__module__.startswith("vllm.")


def _is_moe_router(parent, name, module) -> bool:
    """The expert-selection projection of a sparse-MoE block: a Linear called ``gate`` / ``router`` beside an
    ``experts`` container, or any Linear subclass named ``*Router``."""
    if type(module).__name__.endswith("Router"):
        return True
    return name in ("gate", "router") and hasattr(parent, "experts") and isinstance(module, nn.Linear)


def _linear_weight(module) -> torch.Tensor:
    """The ``[out, in]`` weight of a module ``is_linear_module`` accepted (Conv1D stores the transpose)."""
    w = module.weight.data
    if module.__class__.__name__ == "Conv1D":
        w = w.t().contiguous()
    return w


def convert_gptq(module, awq=False, llm_awq=False, act_order=False):
    """GPTQ / AWQ int4 tensors -> canonical asym_int4 blocks ``[d | m | qs]`` with ``m = -(zero * scale)``,
    low nibble = first half of the 64-group (reference convert.py:379-453)."""
    from ..transformers.awq.linear import unpack_awq, unpack_gptq
    if awq:
        weight, zeros = unpack_awq(module.qweight, module.qzeros, module.w_bit, llm_awq)
    else:
        weight, zeros = unpack_gptq(module.qweight, module.qzeros, module.bits)
    scales = module.scales.float()
    # weight: [out, in] codes 0..15 ; zeros, scales: [in/group, out]
    out_f, in_f = weight.shape
    group = in_f // scales.shape[0]
    if group % 64 != 0:
        raise ValueError("group_size must be a multiple of 64 to repack into asym_int4 blocks")
    if act_order and hasattr(module, "g_idx"):
        pass  # activation reordering is applied on the input (LowBitLinear.act_order)
    rep = group // 64
    scales64 = scales.t().contiguous().repeat_interleave(rep, dim=1)          # [out, in/64]
    zeros64 = zeros.t().contiguous().float().repeat_interleave(rep, dim=1)    # [out, in/64]
    d = scales64.to(torch.float16)
    m = (-(zeros64 * scales64)).to(torch.float16)
    w = weight.view(out_f, in_f // 64, 64).to(torch.uint8)
    qs = (w[:, :, :32] | (w[:, :, 32:] << 4)).to(torch.uint8)
    blocks = torch.cat([d.unsqueeze(-1).view(torch.uint8), m.unsqueeze(-1).view(torch.uint8), qs], dim=-1)
    return blocks.reshape(-1).contiguous()


def use_scale_search(model_config, qtype):
    if qtype == qt.FP6 and getattr(model_config, "model_type", None) not in ("qwen2",):
        return True
    if qtype == qt.FP8E4 and getattr(model_config, "model_type", None) not in ("chatglm",):
        if getattr(model_config, "model_type", None) == "llama" and getattr(model_config, "vocab_size", 0) == 128256:
            return False
        return True
    return False


def _make_low_bit(module, name, in_features, out_features, mp_group, cur_qtype, cur_imatrix, model_config,
                  convert_shape_only, device, optimize_lm_head, enable_scale_search, act_order):
    has_bias = getattr(module, "bias", None) is not None
    # vLLM's parallel linears return ``(output, output_bias)``; their replacements keep that contract
    # (reference convert.py:538-560 picks vLLMLowBitLinear for them)
    cls = vLLMLowBitLinear if _is_vllm_linear(module) else LowBitLinear
    new_linear = cls(in_features, out_features, cur_qtype, has_bias, mp_group=mp_group,
                     optimize_lm_head=optimize_lm_head, act_order=act_order,
                     enable_scale_search=enable_scale_search)
    if is_gptq_linear(module) or module.__class__.__name__ == "WQLinear_GEMM":
        awq = module.__class__.__name__ == "WQLinear_GEMM"
        packed = convert_gptq(module, awq=awq, llm_awq=getattr(module, "backend", "") == "llm-awq",
                              act_order=act_order)
        new_linear._parameters["weight"] = FP4Params(packed, requires_grad=False, quantized=True,
                                                     _shape=torch.Size((out_features, in_features)),
                                                     qtype=cur_qtype).to(device)
    else:
        w = _linear_weight(module)
        param = FP4Params(w, requires_grad=False, quantized=False, _shape=None,
                          convert_shape_only=convert_shape_only, qtype=cur_qtype, imatrix=cur_imatrix,
                          in_features=in_features, enable_scale_search=enable_scale_search)
        new_linear._parameters["weight"] = param.to(device)
    if has_bias:
        new_linear._parameters["bias"] = nn.Parameter(module.bias.data.to(device) if str(device) != "meta"
                                                      else module.bias.data, requires_grad=False)
    return new_linear


def _replace_with_low_bit_linear(model, qtype, modules_to_not_convert=None, convert_shape_only=False,
                                 cpu_embedding=False, prefix_name="", imatrix_data=None, embedding_qtype=None,
                                 model_config=None, torch_dtype=torch.float32, mixed_precision=False,
                                 act_order=False, enable_scale_search=False, device="cpu", materialize=None):
    """Recursive swap (reference convert.py:469-748).  Returns ``(model, has_been_replaced)``."""
    has_been_replaced = False
    for name, module in list(model.named_children()):
        full_name = prefix_name + "." + name if prefix_name else name
        if materialize is not None:
            materialize(module, full_name)
        is_linear, (in_features, out_features, mp_group) = is_linear_module(module)
        skip = modules_to_not_convert is not None and any(k in full_name for k in modules_to_not_convert)
        if skip and not isinstance(module, nn.Embedding):
            # substring match on the dotted name (reference convert.py:489-491)
            continue
        if is_linear and _is_moe_router(model, name, module):
            # routers stay in full precision: their modeling code multiplies by ``.weight`` directly or carries the
            # top-k selection in a Linear subclass (the reference keeps them out per family, convert.py:1100-1135)
            continue
        if is_fused_experts(module) and qtype not in qt.FLOAT_QTYPES:
            new_mod = convert_fused_experts(module, qtype, device=device, convert_shape_only=convert_shape_only,
                                            enable_scale_search=enable_scale_search)
            model._modules[name] = new_mod
            has_been_replaced = True
            continue
        if is_linear and not isinstance(module, LowBitLinear):
            optimize_lm_head = is_lm_head(name, model_config, out_features) and \
                os.environ.get("IPEX_LLM_LAST_LM_HEAD", "1") != "0"
            if qtype not in qt.FLOAT_QTYPES:
                cur_qtype, cur_imatrix = get_cur_qtype_and_imatrix(qtype, full_name, imatrix_data, model_config)
                # mixed precision: lm_head keeps more bits when the body is int4 (reference convert.py:618-622)
                if mixed_precision and is_lm_head(name, model_config, out_features):
                    if cur_qtype in (qt.SYM_INT4, qt.ASYM_INT4):
                        cur_qtype = qt.SYM_INT8 if in_features % 256 != 0 else qt.Q6_K
                block = get_block_size(cur_qtype)
                if in_features % 64 != 0 or in_features % block != 0:
                    # kernels need whole blocks along K: leave this layer unquantized (reference convert.py:611-613)
                    logger.info("%s: in_features %d is not a multiple of the block size, kept in %s",
                                full_name, in_features, torch_dtype)
                    continue
                new_linear = _make_low_bit(module, name, in_features, out_features, mp_group, cur_qtype, cur_imatrix,
                                           model_config, convert_shape_only, device, optimize_lm_head,
                                           enable_scale_search or use_scale_search(model_config, cur_qtype),
                                           act_order)
            else:
                cls = FP16Linear if qtype == qt.FP16 else BF16Linear
                if _is_vllm_linear(module):
                    cls = vLLMFP16Linear if qtype == qt.FP16 else vLLMBF16Linear
                has_bias = getattr(module, "bias", None) is not None
                new_linear = cls(in_features, out_features, has_bias, mp_group=mp_group,
                                 optimize_lm_head=optimize_lm_head)
                dt = torch.float16 if qtype == qt.FP16 else torch.bfloat16
                new_linear.weight = nn.Parameter(_linear_weight(module).to(dt), requires_grad=False)
                if has_bias:
                    new_linear.bias = nn.Parameter(module.bias.data.to(dt), requires_grad=False)
                if str(device) not in ("cpu", "meta"):
                    new_linear = new_linear.to(device)
            new_linear.requires_grad_(False)
            if getattr(module, "gather_output", False):
                new_linear.tp_gather = getattr(module, "tp_group", None)     # vocabulary-parallel lm_head
            model._modules[name] = new_linear
            has_been_replaced = True
            continue
        if isinstance(module, nn.Embedding) and (type(module) is nn.Embedding or hasattr(module, "scalar_embed_scale")):
            new_emb = None
            if embedding_qtype is not None and not skip:
                q = embedding_qtype if isinstance(embedding_qtype, int) else qt.qtype_from_name(embedding_qtype)
                new_emb = LowBitEmbedding.from_embedding(module, q, convert_shape_only, device)
                has_been_replaced = True
            elif cpu_embedding:
                new_emb = CPUEmbedding.from_embedding(module)
            if new_emb is not None:
                if hasattr(module, "scalar_embed_scale"):          # Gemma family: rows are scaled after the look-up
                    new_emb.embed_scale_value = float(module.scalar_embed_scale)
                model._modules[name] = new_emb
            continue
        if len(list(module.children())) > 0:
            _, flag = _replace_with_low_bit_linear(module, qtype, modules_to_not_convert, convert_shape_only,
                                                   cpu_embedding, full_name, imatrix_data, embedding_qtype,
                                                   model_config, torch_dtype, mixed_precision, act_order,
                                                   enable_scale_search, device, materialize)
            has_been_replaced = has_been_replaced or flag
    return model, has_been_replaced


def replace_with_low_bit_linear_for_module(model, qtype, module_name=None, modules_to_not_convert=None,
                                           current_key_name=None, convert_shape_only=False,
                                           torch_dtype="auto"):
    """Convert one named sub-module in place (ReLoRA re-quantization uses this)."""
    parent, leaf = model, module_name
    if module_name and "." in module_name:
        path = module_name.split(".")
        for p in path[:-1]:
            parent = getattr(parent, p)
        leaf = path[-1]
    holder = nn.Module()
    holder._modules[leaf] = getattr(parent, leaf)
    _replace_with_low_bit_linear(holder, qtype, modules_to_not_convert, convert_shape_only,
                                 model_config=getattr(model, "config", None))
    parent._modules[leaf] = holder._modules[leaf]
    return model


# ------------------------------------------------------------------------------------------------
# forward replacement helpers
# ------------------------------------------------------------------------------------------------
def _class_matches(module, target) -> bool:
    if isinstance(target, str):
        return module.__class__.__name__ == target
    return module.__class__ == target


def convert_forward(m, target_m, new_forward):
    """Bind ``new_forward`` as ``forward`` on every sub-module of class ``target_m`` (class or class name)."""
    if _class_matches(m, target_m):
        m.forward = types.MethodType(new_forward, m)
    for _, sub_m in m.named_children():
        convert_forward(sub_m, target_m, new_forward)


def replace_func(m, target_m, func_name, new_func):
    if _class_matches(m, target_m):
        setattr(m, func_name, types.MethodType(new_func, m))
    for _, sub_m in m.named_children():
        replace_func(sub_m, target_m, func_name, new_func)


def replace_attr(m, target_m, attr_name, value):
    if _class_matches(m, target_m):
        setattr(m, attr_name, value)
    for _, sub_m in m.named_children():
        replace_attr(sub_m, target_m, attr_name, value)


def convert_bigdl_other_module(model, dtype):
    """Cast every floating leaf that is not a packed weight to ``dtype`` (reference convert.py:1141)."""
    for module in model.modules():
        if isinstance(module, (LowBitLinear, LowBitEmbedding, CPUEmbedding, DiskEmbedding)):
            if isinstance(module, LowBitLinear) and module.bias is not None:
                module.bias.data = module.bias.data.to(dtype)
            continue
        if isinstance(module, LowBitExperts):
            continue
        for pname, p in list(module._parameters.items()):
            if p is not None and not isinstance(p, FP4Params) and p.is_floating_point():
                p.data = p.data.to(dtype)
        for bname, b in list(module._buffers.items()):
            if b is not None and b.is_floating_point() and "inv_freq" not in bname:
                module._buffers[bname] = b.to(dtype)


# ------------------------------------------------------------------------------------------------
# pre / post optimisation, driven by the family registry
# ------------------------------------------------------------------------------------------------
def _required_forward_fixes(model):
    """Forward replacements that a packed model needs to be correct at all, applied even when the optimisations are
    switched off: the T5 line's feed-forward casts its activations to ``wo.weight.dtype``, which is a byte type for
    a packed weight."""
    from ..models.common import t5_dense_forward
    for mod in model.modules():
        if type(mod).__name__.endswith(("DenseActDense", "DenseGatedActDense")) and hasattr(mod, "wo") and \
                isinstance(getattr(mod.wo, "weight", None), FP4Params):
            mod.forward = types.MethodType(t5_dense_forward, mod)


def _optimize_pre(model, qtype=None):
    from ..models.registry import family_for
    fam = family_for(model)
    if fam is not None:
        for fn in fam.pre:
            model.apply(lambda mod, fn=fn: fn(mod, model.config))
    # composite models: re-enter on the inner language model
    for inner_name in ("language_model", "llm"):
        inner = getattr(model, inner_name, None)
        if inner is not None and hasattr(inner, "config") and inner is not model and fam is None:
            _optimize_pre(inner, qtype)
    return model


def _optimize_post(model):
    from ..models.common import layer_norm_forward, use_attention_interface
    from ..models.registry import family_for
    convert_forward(model, nn.LayerNorm, layer_norm_forward)
    # Attention classes without a forward of their own reach the package's SDPA through the interface registry.
    # Falcon and MPT build their position bias outside that contract and keep their own attention path.
    if os.environ.get("IPEX_LLM_ATTN_INTERFACE", "1") != "0" and \
            getattr(getattr(model, "config", None), "model_type", None) not in ("falcon", "mpt"):
        use_attention_interface(model)
    fam = family_for(model)
    if fam is not None:
        for target, fwd in fam.post:
            convert_forward(model, target, fwd)
        for target, attr, value in fam.attrs:
            replace_attr(model, target, attr, value)
        if fam.post_hook is not None:
            fam.post_hook(model)
    else:
        for inner_name in ("language_model", "llm"):
            inner = getattr(model, inner_name, None)
            if inner is not None and hasattr(inner, "config") and inner is not model:
                _optimize_post(inner)
    return model


def ggml_convert_low_bit(model, qtype, optimize_model=True, convert_shape_only=False, device="cpu",
                         modules_to_not_convert=None, cpu_embedding=False, torch_dtype="auto",
                         imatrix_data=None, embedding_qtype=None, mixed_precision=False,
                         disable_optimize_pre=False, materialize=None):
    """The conversion entry point (reference convert.py:1079-1171)."""
    if qtype in qt.ggml_tensor_qtype.values():
        index = list(qt.ggml_tensor_qtype.values()).index(qtype)
        logger.info("Converting the current model to %s format......", list(qt.ggml_tensor_qtype.keys())[index])
    modules_to_not_convert = [] if modules_to_not_convert is None else list(modules_to_not_convert)
    model_config = getattr(model, "config", None)
    model_type = getattr(model_config, "model_type", None)

    enable_scale_search = use_scale_search(model_config, qtype)
    act_order = False
    qc = getattr(model_config, "quantization_config", None)
    if qc is not None:
        act_order = bool(qc.get("desc_act", False)) if isinstance(qc, dict) else bool(getattr(qc, "desc_act", False))

    if optimize_model and not disable_optimize_pre:
        model = _optimize_pre(model, qtype)

    if torch_dtype == "auto" or torch_dtype is None:
        torch_dtype = getattr(model_config, "torch_dtype", None) or getattr(model_config, "dtype", None) \
            or torch.float32
        if isinstance(torch_dtype, str):
            torch_dtype = getattr(torch, torch_dtype, torch.float32)

    model, has_been_replaced = _replace_with_low_bit_linear(
        model, qtype, modules_to_not_convert, convert_shape_only, cpu_embedding, imatrix_data=imatrix_data,
        embedding_qtype=embedding_qtype, model_config=model_config, torch_dtype=torch_dtype,
        mixed_precision=mixed_precision, act_order=act_order, enable_scale_search=enable_scale_search,
        device=device, materialize=materialize)
    if not has_been_replaced:
        warnings.warn("No linear modules were found in your model, it will fall back to the original model.")
    elif str(device) == "cpu":
        if not (getattr(model, "quantization_method", None) == "gptq"):
            if torch_dtype in (torch.float16, torch.bfloat16) and os.environ.get("IPEX_LLM_KEEP_HALF_ON_CPU") != "1":
                convert_bigdl_other_module(model, torch.float32)
    elif str(device) == "meta":
        pass
    else:
        convert_bigdl_other_module(model, torch_dtype if torch_dtype in (torch.float16, torch.bfloat16)
                                   else torch.float16)
        model = model.to(device)

    if optimize_model:
        model = _optimize_post(model)
    elif has_been_replaced:
        _required_forward_fixes(model)
    if hasattr(model, "config") and model_type is not None:
        model._ipex_low_bit = qtype
    return model


def convert_model_hybrid(model):
    """DeepSeek-V3 CPU+GPU split of the reference (convert.py:2045-2069) exists because a 16-GB Arc cannot
    hold the experts; a 180-GB B200 holds them, so the whole model stays on the GPU and this is the identity."""
    return model


def get_enable_ipex():
    return False
