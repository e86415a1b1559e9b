"""``AutoModel*`` API: ``from_pretrained`` / ``load_convert`` / ``save_low_bit`` / ``load_low_bit`` / ``from_gguf``.

Counterpart of python/llm/src/ipex_llm/transformers/model.py of the reference (``save_low_bit`` :59-103,
``_BaseAutoModelClass`` :106-785, the ten Auto classes :788-830).  Same keyword arguments, same on-disk
artefacts (``pytorch_model.bin`` [+ index], ``config.json`` with ``bigdl_transformers_low_bit``,
``generation_config.json``, ``load_keys.json``).

B200-first additions:
* ``device="cuda"`` (or ``device_map="cuda"``) quantizes on the GPU, layer by layer, straight into the
  tensor-core tile layout instead of packing on the host and converting afterwards;
* ``from_config`` builds a random-initialised model of a given architecture directly in low-bit form on the
  GPU (what the benchmarks use: there is no checkpoint to download on an air-gapped box).
"""
from __future__ import annotations

import copy
import json
import logging
import os
import types
import warnings
from contextlib import contextmanager

import torch
import transformers
from transformers.configuration_utils import PretrainedConfig

from ..quant import qtypes as qt
from ..quant.params import FP4Params
from ..quant.policy import load_imatrix_data
from ..utils.common import invalidInputError
from .convert import ggml_convert_low_bit

logger = logging.getLogger(__name__)

WEIGHTS_NAME = "pytorch_model.bin"
WEIGHTS_INDEX_NAME = "pytorch_model.bin.index.json"
LOAD_KEYS_NAME = "load_keys.json"


# ------------------------------------------------------------------------------------------------
# serialization
# ------------------------------------------------------------------------------------------------
def _plain_state_dict(model):
    """State dict with packed weights as plain (canonical, CPU) tensors."""
    out = {}
    # keep_vars: the FP4Params objects themselves (a detached copy would lose qtype / shape, and with them the
    # knowledge that GPU-resident bytes are in tile order and must go back to canonical blocks)
    for k, v in model.state_dict(keep_vars=True).items():
        if isinstance(v, FP4Params) and v.quantized:
            v = v.to("cpu") if v.data.device.type != "cpu" else v
            out[k] = v.data.detach().clone()
        else:
            out[k] = v.detach().to("cpu")
    return out


def _parse_size(s):
    if isinstance(s, int):
        return s
    s = s.upper().strip()
    for suf, mul in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if s.endswith(suf):
            return int(float(s[:-2]) * mul)
    return int(s)


def save_low_bit(self, save_directory, max_shard_size="10GB", **kwargs):
    """Write a low-bit checkpoint: the packed weights exactly as held in memory (canonical block layout),
    the config with ``bigdl_transformers_low_bit`` and the list of keys (``load_keys.json``)."""
    invalidInputError(self.config.to_dict().get("bigdl_transformers_low_bit", False),
                      "Detected this model is not a low-bit model, please use from_pretrained's"
                      " load_in_4bit or load_in_low_bit parameter to load a 4-bit model first.")
    if hasattr(self.config, "quantization_config"):
        delattr(self.config, "quantization_config")
        if hasattr(self.config, "_pre_quantization_dtype"):
            delattr(self.config, "_pre_quantization_dtype")
    os.makedirs(save_directory, exist_ok=True)
    if self.config.to_dict().get("bigdl_transformers_low_bit") in ("mixed_fp4", "mixed_fp8"):
        # every layer chose between an integer and a float format of the same size by its own error: the bytes do
        # not say which, so the choice is written down for load_low_bit
        chosen = {n: qt.qtype_name(m.weight.qtype) for n, m in self.named_modules()
                  if isinstance(getattr(m, "weight", None), FP4Params) and m.weight.quantized}
        self.config.update({"bigdl_layer_qtypes": chosen})
    disk_embedding = getattr(self.config, "bigdl_disk_embedding", False)
    if disk_embedding:
        from ..ops.embedding import DiskEmbedding
        self.apply(DiskEmbedding.restore_normal_embedding)
    sd = _plain_state_dict(self)
    if disk_embedding:
        from ..ops.embedding import DiskEmbedding
        self.apply(DiskEmbedding.replace_normal_embedding)

    limit = _parse_size(max_shard_size)
    shards, cur, cur_size = [], {}, 0
    for k, v in sd.items():
        nbytes = v.numel() * v.element_size()
        if cur and cur_size + nbytes > limit:
            shards.append(cur)
            cur, cur_size = {}, 0
        cur[k] = v
        cur_size += nbytes
    shards.append(cur)
    if len(shards) == 1:
        torch.save(shards[0], os.path.join(save_directory, WEIGHTS_NAME))
    else:
        weight_map = {}
        for i, shard in enumerate(shards):
            fname = f"pytorch_model-{i + 1:05d}-of-{len(shards):05d}.bin"
            torch.save(shard, os.path.join(save_directory, fname))
            for k in shard:
                weight_map[k] = fname
        total = sum(v.numel() * v.element_size() for v in sd.values())
        with open(os.path.join(save_directory, WEIGHTS_INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)

    self.config.save_pretrained(save_directory)
    if getattr(self, "can_generate", lambda: False)() and getattr(self, "generation_config", None) is not None:
        self.generation_config.save_pretrained(save_directory)
    with open(os.path.join(save_directory, LOAD_KEYS_NAME), "w") as f:
        json.dump({"all_checkpoint_keys": list(sd.keys())}, f)


def _load_state_dict_from_dir(path):
    index = os.path.join(path, WEIGHTS_INDEX_NAME)
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = [WEIGHTS_NAME]
    sd = {}
    for fn in files:
        fp = os.path.join(path, fn)
        invalidInputError(os.path.exists(fp), f"checkpoint shard {fp} is missing")
        sd.update(torch.load(fp, map_location="cpu", weights_only=True))
    return sd


@contextmanager
def _meta_init():
    """Build modules without allocating or initialising weights."""
    try:
        from transformers.initialization import no_init_weights
    except ImportError:  # older transformers
        from transformers.modeling_utils import no_init_weights
    try:
        ctx = no_init_weights()
    except TypeError:
        ctx = no_init_weights(True)
    with ctx, torch.device("meta"):
        yield


def _rebuild_nonpersistent(model, device="cpu"):
    """Buffers that are computed in ``__init__`` and not stored in checkpoints were built on ``meta`` (or left
    uninitialised by ``to_empty``): re-create them for real.  Rotary embeddings are re-instantiated from their config;
    scaled word embeddings (Gemma family: ``embed_scale = sqrt(hidden)``) get their scalar back."""
    for name, mod in list(model.named_modules()):
        if "embed_scale" in getattr(mod, "_non_persistent_buffers_set", ()) and hasattr(mod, "scalar_embed_scale"):
            mod._buffers["embed_scale"] = torch.tensor(float(mod.scalar_embed_scale), device=device)
            continue
        if "RotaryEmbedding" in type(mod).__name__ and hasattr(mod, "config"):
            try:
                new = type(mod)(config=mod.config)
            except TypeError:
                continue
            parent = model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            parent._modules[parts[-1]] = new.to(device)
            continue
        # any other module with buffers that no checkpoint holds and that still sit on ``meta`` (GPT-J's sinusoidal
        # table, ...): build one fresh instance of that module alone and take its buffers
        lost = [b for b in getattr(mod, "_non_persistent_buffers_set", ())
                if mod._buffers.get(b) is not None and mod._buffers[b].device.type == "meta"]
        if lost:
            fresh = None
            attempts = []
            configs = [mod.config] if hasattr(mod, "config") else []
            # modules that do not keep their config (BERT's embeddings): the config of the nearest owner up the tree
            parts = name.split(".")
            for depth in range(len(parts) - 1, -1, -1):
                owner = model.get_submodule(".".join(parts[:depth])) if depth else model
                if hasattr(owner, "config") and all(owner.config is not c for c in configs):
                    configs.append(owner.config)
            for c in configs:
                attempts += [((c, getattr(mod, "layer_idx", None)), {}), ((c,), {})]
            # small helper modules (vision rotary tables, ...) keep their constructor arguments as attributes
            import inspect
            try:
                names = [p for p in inspect.signature(type(mod).__init__).parameters if p != "self"]
                if names and all(hasattr(mod, n) for n in names):
                    attempts.append(((), {n: getattr(mod, n) for n in names}))
            except (TypeError, ValueError):
                pass
            for args, kwargs in attempts:
                try:
                    with torch.device("cpu"):
                        fresh = type(mod)(*args, **kwargs)
                    break
                except Exception:  # noqa: BLE001 - another constructor signature
                    continue
            invalidInputError(fresh is not None, f"cannot rebuild the buffers {lost} of {name} ({type(mod).__name__})")
            for b in lost:
                mod._buffers[b] = fresh._buffers[b].to(device)


def _materialize_meta(model, device, dtype, seed=0, std=0.02):
    """Give every remaining ``meta`` parameter/buffer real storage on ``device`` (random normal weights,
    ones for norm scales, zeros for biases)."""
    gen = torch.Generator(device=device if str(device) != "cpu" else "cpu")
    gen.manual_seed(seed)
    for mod in model.modules():
        for pname, p in list(mod._parameters.items()):
            if p is None or p.device.type != "meta" or isinstance(p, FP4Params):
                continue
            shape = tuple(p.shape)
            if p.dim() == 1:
                is_norm = "norm" in type(mod).__name__.lower() or pname == "weight" and "Norm" in type(mod).__name__
                t = torch.ones(shape, dtype=dtype, device=device) if (is_norm and pname == "weight") \
                    else torch.zeros(shape, dtype=dtype, device=device)
            else:
                t = torch.empty(shape, dtype=dtype, device=device).normal_(0.0, std, generator=gen)
            mod._parameters[pname] = torch.nn.Parameter(t, requires_grad=False)
        for bname, b in list(mod._buffers.items()):
            if b is not None and b.device.type == "meta":
                mod._buffers[bname] = torch.zeros(b.shape, dtype=b.dtype, device=device)


def _attach_api(model, qtype_name=None):
    from .generation import ipex_generate
    model.save_low_bit = types.MethodType(save_low_bit, model)
    if hasattr(model, "generate") and not getattr(model, "_ipex_generate_patched", False):
        model._hf_generate = model.generate
        model.generate = types.MethodType(ipex_generate, model)
        model._ipex_generate_patched = True
        from ..engine import decode_step_host, prefill_host
        model.decode_step = types.MethodType(decode_step_host, model)
        model.prefill = types.MethodType(prefill_host, model)
    return model


class _BaseAutoModelClass:
    HF_Model = None

    # -- from_pretrained ------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, *args, **kwargs):
        """Load a Hugging Face checkpoint and convert it to low-bit form.

        Keyword arguments (same as the reference, model.py:111-388): ``load_in_4bit``, ``load_in_low_bit``
        (``sym_int4 | asym_int4 | sym_int5 | asym_int5 | sym_int8 | nf3 | nf4 | fp4 | fp6 | fp8 | fp8_e4m3 |
        fp8_e5m2 | fp16 | bf16 | q2_k | q4_k | q5_k | q6_k | gguf_q4k_s | gguf_q4k_m | mixed_fp4 | mixed_fp8``),
        ``optimize_model``, ``modules_to_not_convert``, ``speculative``, ``cpu_embedding``, ``disk_embedding``,
        ``imatrix``, ``model_hub``, ``embedding_qtype``, ``mixed_precision``, ``pipeline_parallel_stages``,
        ``quantization_config`` (BitsAndBytes / GPTQ / AWQ), ``torch_dtype``; plus ``device`` (B200 addition).
        """
        pretrained_model_name_or_path = kwargs.get("pretrained_model_name_or_path", None) \
            if len(args) == 0 else args[0]
        model_hub = kwargs.pop("model_hub", "huggingface")
        invalidInputError(model_hub in ["huggingface", "modelscope"],
                          "The parameter `model_hub` is supposed to be `huggingface` or `modelscope`, "
                          f"but got {model_hub}.")
        invalidInputError(model_hub == "huggingface", "modelscope is not installed in this environment")
        config_dict, _ = PretrainedConfig.get_config_dict(pretrained_model_name_or_path)
        invalidInputError(not config_dict.get("bigdl_transformers_low_bit", False),
                          f"Detected model is a low-bit({config_dict.get('bigdl_transformers_low_bit')}) model, "
                          "Please use load_low_bit to load this model.")

        load_in_4bit = kwargs.pop("load_in_4bit", False)
        load_in_low_bit = kwargs.pop("load_in_low_bit", None)
        optimize_model = kwargs.pop("optimize_model", True)
        user_quantization_config = kwargs.pop("quantization_config", None)
        speculative = kwargs.pop("speculative", False)
        pipeline_parallel_stages = kwargs.pop("pipeline_parallel_stages", 1)
        torch_dtype = kwargs.pop("torch_dtype", kwargs.pop("dtype", None))
        embedding_qtype = kwargs.pop("embedding_qtype", None)

        # BitsAndBytesConfig mapping (reference model.py:194-234)
        if user_quantization_config is not None and \
                "BitsAndBytesConfig" in str(user_quantization_config.__class__):
            qc = user_quantization_config
            if getattr(qc, "bnb_4bit_quant_type", None) is not None:
                bnb_4bit_type = qc.bnb_4bit_quant_type
                if bnb_4bit_type == "nf4":
                    load_in_low_bit = "nf4"
                elif bnb_4bit_type == "fp4":
                    warnings.warn("BigDL LLM QLoRA does not support fp4 now, use default nf4", FutureWarning)
                    load_in_low_bit = "nf4"
                elif bnb_4bit_type == "int4":
                    load_in_low_bit = "sym_int4"
                else:
                    invalidInputError(False, "Only nf4 or int4 is supported for bnb_4bit_quant_type")
            else:
                warnings.warn("bnb_4bit_quant_type is None, use default int4", FutureWarning)
                load_in_low_bit = "sym_int4"
            if getattr(qc, "bnb_4bit_use_double_quant", False):
                # same behaviour as the reference (model.py:215-218): nf4 keeps one fp16 scale per 64-group
                warnings.warn("double quantization of the nf4 scales is not supported, set to False", FutureWarning)
            if qc.bnb_4bit_compute_dtype is not None:
                bnb_dtype = qc.bnb_4bit_compute_dtype
                invalidInputError(bnb_dtype in (torch.float32, torch.bfloat16),
                                  "Only float32 or bfloat16 is supported for bnb_4bit_compute_dtype")
                if torch_dtype is None:
                    torch_dtype = bnb_dtype
            optimize_model = False
            kwargs["modules_to_not_convert"] = ["lm_head"]
            user_quantization_config = None
            load_in_4bit = False

        if load_in_4bit or load_in_low_bit:
            if config_dict.get("quantization_config", None) is not None:
                q_config = config_dict["quantization_config"]
                method = q_config.get("quant_method")
                if method == "gptq":
                    invalidInputError(q_config["bits"] == 4 or load_in_low_bit == "asym_int4" or True,
                                      "Only 4-bit gptq is supported.")
                    invalidInputError(q_config["group_size"] % 64 == 0, "group_size must be divisible by 64.")
                    load_in_low_bit = "asym_int4"
                    kwargs["_gptq"] = q_config
                elif method == "awq":
                    invalidInputError(q_config["bits"] == 4, "Only 4-bit awq is supported.")
                    invalidInputError(q_config["version"] == "gemm", "Only gemm version is supported.")
                    invalidInputError(q_config["zero_point"], "Only awq zero_point = True is supported.")
                    load_in_low_bit = "asym_int4"
                    kwargs["_awq"] = q_config
            q_k = load_in_low_bit if load_in_low_bit else "sym_int4"
            model = cls.load_convert(q_k, optimize_model, *args, torch_dtype=torch_dtype,
                                     embedding_qtype=embedding_qtype, **kwargs)
            if pipeline_parallel_stages > 1:
                from ..parallel.pp import pipeline_parallel
                if speculative:
                    invalidInputError(False, "Please do not set speculative=True when using pipeline_parallel_stages")
                invalidInputError(torch.distributed.is_initialized() and
                                  torch.distributed.get_world_size() == pipeline_parallel_stages,
                                  "Please make sure world size is same as `pipeline_parallel_stages`")
                model = pipeline_parallel(model, pipeline_parallel_stages, torch_dtype or model.dtype)
                torch.distributed.barrier()
            if speculative:
                from .speculative import attach_draft_model
                # the target keeps half precision weights; the draft is a sym_int4 copy of the same checkpoint
                draft = cls.load_convert("sym_int4", optimize_model, *args, torch_dtype=torch_dtype, **kwargs)
                attach_draft_model(model, draft)
        else:
            extra = {}
            if torch_dtype is not None:
                extra["dtype"] = torch_dtype
            from .remote_archs import maybe_load_remote_arch
            model = maybe_load_remote_arch(pretrained_model_name_or_path, extra.get("dtype"))
            if model is None:
                model = cls.HF_Model.from_pretrained(*args, **extra, **_strip_private(kwargs))
        return _attach_api(model)

    @classmethod
    def load_convert(cls, q_k, optimize_model, *args, **kwargs):
        invalidInputError(q_k in qt.ggml_tensor_qtype or q_k in qt.gguf_mixed_qtype,
                          f"Unknown load_in_low_bit value: {q_k}, expected:"
                          f" sym_int4, asym_int4, sym_int5, asym_int5, sym_int8, nf3, nf4, "
                          f"fp4, fp6, fp8, fp8_e4m3, fp8_e5m2, fp16,  bf16, gguf_iq2_xxs, "
                          f"gguf_iq2_xs, gguf_iq1_s, gguf_q4k_m, gguf_q4k_s, q2_k, q4_k, q6_k, "
                          f"mixed_fp4 or mixed_fp8.")
        if q_k.endswith("_rtn"):
            # per-channel round-to-nearest containers belong to the NPU entry point of the reference; the same
            # request here takes the blocked format of the same width, as ``transformers.npu_model`` does
            warnings.warn(f"{q_k} is a per-channel NPU format; using {q_k[:-4]} blocks instead", UserWarning)
            q_k = q_k[:-4]
        qtype = qt.qtype_from_name(q_k)
        imatrix_file = kwargs.pop("imatrix", None)
        if q_k in ("gguf_iq2_xxs", "gguf_iq2_xs", "gguf_iq1_s"):
            invalidInputError(imatrix_file is not None,
                              "For gguf_iq2 and gguf_iq1 quantization, imatrix is needed.")
        cpu_embedding = kwargs.get("cpu_embedding", False)
        embedding_qtype = kwargs.pop("embedding_qtype", None)
        if q_k in ("gguf_iq2_xxs", "gguf_iq2_xs", "gguf_iq1_s", "q2_k") and not cpu_embedding:
            embedding_qtype = "q2_k"
        elif q_k in ("gguf_q4k_s", "gguf_q4k_m") and not cpu_embedding:
            embedding_qtype = "q4_k"
        if embedding_qtype is not None and not isinstance(embedding_qtype, int):
            embedding_qtype = qt.qtype_from_name(embedding_qtype)
        imatrix_data = load_imatrix_data(imatrix_file) if imatrix_file is not None else None
        mixed_precision = kwargs.pop("mixed_precision", False)
        modules_to_not_convert = kwargs.pop("modules_to_not_convert", [])
        cpu_embedding = kwargs.pop("cpu_embedding", False)
        disk_embedding = kwargs.pop("disk_embedding", False)
        device = kwargs.pop("device", None)
        device_map = kwargs.pop("device_map", None)
        if device is None and isinstance(device_map, str) and device_map.startswith("cuda"):
            device = device_map
        torch_dtype = kwargs.pop("torch_dtype", None)
        gptq = kwargs.pop("_gptq", None)
        awq = kwargs.pop("_awq", None)
        tp_group = kwargs.pop("tp_group", None)

        hf_kwargs = _strip_private(kwargs)
        hf_kwargs.pop("low_cpu_mem_usage", None)
        if awq is not None:
            model = _load_awq(cls, awq, *args, **hf_kwargs)
        elif gptq is not None:
            model = _load_gptq(cls, gptq, *args, **hf_kwargs)
        else:
            extra = {}
            if torch_dtype is not None and torch_dtype != "auto":
                extra["dtype"] = torch_dtype
            from .remote_archs import maybe_load_remote_arch
            path = args[0] if args else hf_kwargs.get("pretrained_model_name_or_path")
            # ChatGLM / Baichuan / InternLM(2) / Qwen-v1 / MiniCPM / Aquila checkpoints: built natively, their remote
            # modeling code is never executed
            model = maybe_load_remote_arch(path, extra.get("dtype"))
            try:
                if model is None:
                    model = cls.HF_Model.from_pretrained(*args, **extra, **hf_kwargs)
            except NotImplementedError:
                logger.info("Failed to load models with `low_cpu_mem_usage` specified, retrying")
                model = cls.HF_Model.from_pretrained(*args, **extra, **hf_kwargs)
        model.config.update({"bigdl_lcmu_enabled": False})
        if tp_group is not None:
            from ..parallel.tp import auto_tp
            model = auto_tp(model, tp_group)
        model = model.to("cpu")
        model = ggml_convert_low_bit(model, qtype, optimize_model, modules_to_not_convert=modules_to_not_convert,
                                     cpu_embedding=cpu_embedding, torch_dtype=torch_dtype or "auto",
                                     imatrix_data=imatrix_data, embedding_qtype=embedding_qtype,
                                     mixed_precision=mixed_precision, device=device or "cpu")
        model.config.update({"bigdl_transformers_low_bit": q_k, "bigdl_disk_embedding": disk_embedding})
        # enable tie_word_embeddings for MPT only (reference model.py:515-522)
        if model.config.architectures is None or model.config.architectures[0] != "MPTForCausalLM":
            model.config.update({"tie_word_embeddings": False})
        if disk_embedding:
            from ..ops.embedding import DiskEmbedding
            model.apply(DiskEmbedding.replace_normal_embedding)
        return _attach_api(model)

    # -- from_config (B200 addition) ---------------------------------------------------------------------
    @classmethod
    def from_config(cls, config, load_in_low_bit="sym_int4", load_in_4bit=False, optimize_model=True,
                    device="cuda", torch_dtype=torch.float16, seed=0, init_std=0.02, modules_to_not_convert=None,
                    tp_group=None, speculative=False, consistent_tp_shards=False, **kwargs):
        """Random-initialised model of ``config``'s architecture, created layer by layer on ``device`` and
        quantized there (weights ~ N(0, init_std), seeded).  Peak memory = one layer in ``torch_dtype`` plus the
        packed model, so a 70B fp8 model is built on one 180-GB GPU without ever existing in half precision."""
        q_k = "sym_int4" if load_in_4bit and not load_in_low_bit else load_in_low_bit
        qtype = qt.qtype_from_name(q_k)
        config = copy.deepcopy(config)
        with _meta_init():
            model = cls.HF_Model.from_config(config, dtype=torch_dtype) if hasattr(cls.HF_Model, "from_config") \
                else cls.HF_Model(config)
        from .random_init import convert_random_init
        model = convert_random_init(model, qtype, optimize_model, device, torch_dtype, seed, init_std,
                                    modules_to_not_convert or [], tp_group, consistent_shards=consistent_tp_shards)
        model.config.update({"bigdl_transformers_low_bit": q_k, "bigdl_disk_embedding": False,
                             "tie_word_embeddings": False})
        stages = kwargs.pop("pipeline_parallel_stages", 1)
        if stages > 1:
            # every rank builds the same seeded model and keeps its own slice of layers
            from ..parallel.pp import pipeline_parallel
            model = pipeline_parallel(model, stages, torch_dtype, device=torch.device(device))
        model = _attach_api(model)
        if speculative:
            from .speculative import attach_draft_model
            draft = cls.from_config(config, "sym_int4", optimize_model=optimize_model, device=device,
                                    torch_dtype=torch_dtype, seed=seed, init_std=init_std)
            attach_draft_model(model, draft)
        return model

    # -- load_low_bit ------------------------------------------------------------------------------------
    @classmethod
    def load_low_bit(cls, pretrained_model_name_or_path, *model_args, **kwargs):
        """Load a directory written by ``save_low_bit`` (reference model.py:530-785): build the model on
        ``meta``, create empty packed parameters of the right shapes, then assign the tensors."""
        invalidInputError(os.path.isdir(str(pretrained_model_name_or_path)),
                          "load_low_bit expects a local directory written by save_low_bit")
        kwargs.pop("trust_remote_code", None)
        optimize_model = kwargs.pop("optimize_model", True)
        cpu_embedding = kwargs.pop("cpu_embedding", False)
        embedding_qtype = kwargs.pop("embedding_qtype", None)
        torch_dtype = kwargs.pop("torch_dtype", kwargs.pop("dtype", "auto"))
        pipeline_parallel_stages = kwargs.pop("pipeline_parallel_stages", 1)
        mixed_precision = kwargs.pop("mixed_precision", False)
        modules_to_not_convert = kwargs.pop("modules_to_not_convert", [])
        device = kwargs.pop("device", None)
        config_dict, _ = PretrainedConfig.get_config_dict(pretrained_model_name_or_path)
        low_bit = config_dict.pop("bigdl_transformers_low_bit", False)
        invalidInputError(low_bit,
                          "Detect this model is not a low-bit model, Please use from_pretrained"
                          " with load_in_4bit or load_in_low_bit to get a low-bit model , and "
                          " serialize the model using save_low_bit first.")
        invalidInputError(low_bit in qt.ggml_tensor_qtype or low_bit in qt.gguf_mixed_qtype,
                          f"Unknown bigdl_transformers_low_bit value: {low_bit}")
        qtype = qt.qtype_from_name(low_bit)
        if low_bit in ("gguf_iq2_xxs", "gguf_iq2_xs", "gguf_iq1_s", "q2_k") and not cpu_embedding:
            embedding_qtype = "q2_k"
        elif low_bit in ("gguf_q4k_s", "gguf_q4k_m") and not cpu_embedding:
            embedding_qtype = "q4_k"
        if embedding_qtype is not None and not isinstance(embedding_qtype, int):
            embedding_qtype = qt.qtype_from_name(embedding_qtype)

        config = transformers.AutoConfig.from_pretrained(pretrained_model_name_or_path)
        keys_file = os.path.join(pretrained_model_name_or_path, LOAD_KEYS_NAME)
        saved_keys = None
        if os.path.exists(keys_file):
            with open(keys_file) as f:
                saved_keys = set(json.load(f)["all_checkpoint_keys"])
        if torch_dtype == "auto":
            torch_dtype = getattr(config, "dtype", None) or getattr(config, "torch_dtype", None) or torch.float32
            if isinstance(torch_dtype, str):
                torch_dtype = getattr(torch, torch_dtype)
        with _meta_init():
            model = cls.HF_Model.from_config(config, dtype=torch_dtype) if hasattr(cls.HF_Model, "from_config") \
                else cls.HF_Model(config)
        # modules that were skipped at save time (e.g. K not a multiple of 64) stay unquantized: the key list
        # tells which ones hold a packed weight
        model = ggml_convert_low_bit(model, qtype, optimize_model, device="meta", convert_shape_only=True,
                                     modules_to_not_convert=modules_to_not_convert, cpu_embedding=cpu_embedding,
                                     embedding_qtype=embedding_qtype, mixed_precision=mixed_precision,
                                     torch_dtype=torch_dtype)
        for mod_name, q_name in (config_dict.get("bigdl_layer_qtypes") or {}).items():
            try:
                mod = model.get_submodule(mod_name)
            except AttributeError:
                continue
            if isinstance(getattr(mod, "weight", None), FP4Params):
                mod.weight.qtype = qt.qtype_from_name(q_name)
                if hasattr(mod, "qtype"):
                    mod.qtype = mod.weight.qtype
        sd = _load_state_dict_from_dir(pretrained_model_name_or_path)
        if saved_keys is not None:
            missing = saved_keys - set(sd.keys())
            invalidInputError(not missing, f"checkpoint is missing keys listed in load_keys.json: {sorted(missing)[:5]}")
        result = model.load_state_dict(sd, strict=False, assign=True)
        real_missing = [k for k in result.missing_keys if "rotary_emb" not in k and "inv_freq" not in k]
        invalidInputError(not real_missing, f"keys missing from the low-bit checkpoint: {real_missing[:8]}")
        _rebuild_nonpersistent(model, "cpu")
        if hasattr(model, "tie_weights") and getattr(config, "tie_word_embeddings", False):
            # a packed output layer came from the checkpoint as its own matrix: tying it to the embedding again
            # would swap the packed parameter for the float table (T5 style maps do that)
            head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
            if not isinstance(getattr(head, "weight", None), FP4Params):
                model.tie_weights()
        model.eval()
        try:
            model.generation_config = transformers.GenerationConfig.from_pretrained(pretrained_model_name_or_path)
        except Exception:  # noqa: BLE001
            pass
        model.config.update({"bigdl_transformers_low_bit": low_bit})
        if pipeline_parallel_stages > 1:
            from ..parallel.pp import pipeline_parallel
            model = pipeline_parallel(model, pipeline_parallel_stages, torch_dtype)
            torch.distributed.barrier()
        if device is not None:
            model = model.to(device)
        return _attach_api(model)

    # -- from_gguf -----------------------------------------------------------------------------------------
    @staticmethod
    def from_gguf(fpath: str, optimize_model: bool = True, cpu_embedding: bool = False, low_bit: str = "sym_int4"):
        """Load a ``.gguf`` file (llama / mistral / mixtral / baichuan / bloom / falcon / mpt / yuan2 families) and
        return ``(model, tokenizer)``."""
        from .gguf.api import load_gguf_model
        # the loader quantizes each matrix as it is read, so the model arrives converted
        model, tokenizer = load_gguf_model(fpath, dtype=torch.float32 if not torch.cuda.is_available() else torch.half,
                                           low_bit=low_bit)
        model.config.update({"bigdl_transformers_low_bit": low_bit})
        return model, tokenizer


def _strip_private(kwargs):
    return {k: v for k, v in kwargs.items() if not k.startswith("_")}


def _load_awq(cls, q_config, *args, **kwargs):
    from .awq.awq import load_awq_checkpoint
    return load_awq_checkpoint(cls.HF_Model, q_config, *args, **kwargs)


def _load_gptq(cls, q_config, *args, **kwargs):
    from .awq.awq import load_gptq_checkpoint
    return load_gptq_checkpoint(cls.HF_Model, q_config, *args, **kwargs)


class AutoModelForCausalLM(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForCausalLM


class AutoModel(_BaseAutoModelClass):
    HF_Model = transformers.AutoModel


class AutoModelForSpeechSeq2Seq(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForSpeechSeq2Seq


class AutoModelForSeq2SeqLM(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForSeq2SeqLM


class AutoModelForSequenceClassification(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForSequenceClassification


class AutoModelForMaskedLM(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForMaskedLM


class AutoModelForQuestionAnswering(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForQuestionAnswering


class AutoModelForNextSentencePrediction(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForNextSentencePrediction


class AutoModelForMultipleChoice(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForMultipleChoice


class AutoModelForTokenClassification(_BaseAutoModelClass):
    HF_Model = transformers.AutoModelForTokenClassification


class AutoModelForVision2Seq(_BaseAutoModelClass):
    HF_Model = getattr(transformers, "AutoModelForVision2Seq", None) or \
        getattr(transformers, "AutoModelForImageTextToText", transformers.AutoModel)


class Qwen2VLModelForConditionalGeneration(_BaseAutoModelClass):
    HF_Model = getattr(transformers, "Qwen2VLForConditionalGeneration", transformers.AutoModel)
