"""vLLM quantization method "htr" backed by the B200 packed-linear kernels.

Drop-in for htr/vllm_plugin.py:14-138 and :408-413 of the reference: same quantization name, same
`quantization_config` keys, same parameter names (`htr_qweight`, `htr_scales`, `htr_su`, `htr_sv`), same
placement rules for fused shards, and `apply()` forwards to `htr_b200.ops.linear`.  The reference's overlays for
a private runtime (Quark / lm-head / "HC" patches, htr/vllm_plugin.py:153-405) patch modules that upstream vLLM
does not have and are not reproduced.

Importing the module registers the method; `register()` is the `vllm.general_plugins` entry point
(`htr = "htr_b200.vllm_plugin:register"`).  Tensor parallelism is refused exactly as in the reference
(htr/vllm_plugin.py:91); multi-GPU execution of tall linears lives in htr_b200/sharded.py.
"""
import collections
import json
import os
import time

import torch
from torch.nn import Parameter
from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig
from vllm.model_executor.utils import set_weight_attrs

# module-name fragments that stay in their source dtype (htr/vllm_plugin.py:11)
SKIP = ("visual", "vision", "audio", "mtp")

_QKV_INDEX = {"q": 0, "k": 1, "v": 2}


def canon(name):
    """Checkpoint key -> the key used in quantization_config["modules"]: drop ".weight", keep from "layers." on
    (htr/vllm_plugin.py:14-18)."""
    if name.endswith(".weight"):
        name = name[: -len(".weight")]
    at = name.rfind("layers.")
    return name if at < 0 else name[at:]


def _shard_range(sizes, shard_id, unit):
    """Rows [start, start+length) of a fused parameter that shard `shard_id` fills, in multiples of `unit` rows
    (16 for qweight strips, 1 for scales, 8 for sign bytes); htr/vllm_plugin.py:67-80."""
    if shard_id is None:
        members = list(range(len(sizes)))
    elif isinstance(shard_id, str):
        members = [_QKV_INDEX[shard_id]]
    elif isinstance(shard_id, (tuple, list)):
        members = [int(i) for i in shard_id]
    else:
        members = [int(shard_id)]
    if members != list(range(members[0], members[-1] + 1)):
        raise AssertionError(f"HTR: shard ids must be contiguous, got {members}")
    start = sum(sizes[: members[0]])
    length = sum(sizes[i] for i in members)
    if start % unit or length % unit:
        raise AssertionError(f"HTR: shard [{start}, {start + length}) is not a multiple of {unit} rows")
    return start // unit, length // unit


@register_quantization_config("htr")
class HTRConfig(QuantizationConfig):
    """quantization_config = {"quant_method": "htr", "wire": "HTR-W1", "modules": {prefix: {"K": k}}, ...}
    (written by the reference's converter, htr/quantize.py:281-283)."""

    def __init__(self, modules, wire="HTR-W1"):
        super().__init__()
        if wire != "HTR-W1":
            raise AssertionError(wire)
        self.modules = {canon(name): int(spec["K"]) for name, spec in modules.items()}

    def get_name(self):
        return "htr"

    def get_supported_act_dtypes(self):
        return [torch.bfloat16, torch.float16]

    @classmethod
    def get_min_capability(cls):
        return 0

    @staticmethod
    def get_config_filenames():
        return []

    @classmethod
    def from_config(cls, config):
        return cls(config.get("modules", {}), config.get("wire", "HTR-W1"))

    def get_quant_method(self, layer, prefix):
        from vllm.model_executor.layers.vocab_parallel_embedding import ParallelLMHead

        leaf_name = prefix.split(".")[-1]
        if isinstance(layer, ParallelLMHead):
            # only a module literally called lm_head with a configured width is packed; other embeddings are not
            width = self.modules.get("lm_head")
            return HTRLinearMethod(width) if (width is not None and leaf_name == "lm_head") else None
        if not isinstance(layer, LinearBase):
            return None
        if any(tag in prefix.split(".") or tag in prefix for tag in SKIP):
            return UnquantizedLinearMethod()
        parent, _, leaf = canon(prefix).rpartition(".")
        fused = (getattr(self, "packed_modules_mapping", None) or {}).get(leaf, [leaf])
        widths = [self.modules.get(f"{parent}.{part}" if parent else part) for part in fused]
        if all(w is None for w in widths):
            return UnquantizedLinearMethod()
        if None in widths or len(set(widths)) != 1:
            raise ValueError(f"HTR: fused module {prefix} has mixed quantization {dict(zip(fused, widths))}")
        return HTRLinearMethod(widths[0])


class HTRLinearMethod(LinearMethodBase):
    """Creates the four HTR-W1 tensors of a (possibly fused) linear and runs it through htr::linear."""

    def __init__(self, K):
        self.K = K

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size, params_dtype,
                       **extra_weight_attrs):
        n, sizes = input_size_per_partition, list(output_partition_sizes)
        m = sum(sizes)
        assert input_size_per_partition == input_size, "HTR: tensor parallelism is not supported"
        assert n % 128 == 0 and all(s % 128 == 0 for s in sizes), (n, sizes)
        K = self.K
        tensors = {
            "htr_qweight": (torch.empty(m // 16, n // 16, 8 * K, dtype=torch.int32), 16),
            "htr_scales": (torch.empty(m, dtype=torch.float16), 1),
            "htr_sv": (torch.empty(m // 8, dtype=torch.uint8), 8),
        }

        def row_loader(unit):
            def load(param, loaded, shard_id=None):
                if shard_id is None:            # stacked-weight mappers pass the shard as an attribute of the tensor
                    shard_id = getattr(loaded, "shard_id", None)
                start, length = _shard_range(sizes, shard_id, unit)
                assert tuple(loaded.shape) == (length,) + tuple(param.shape[1:]), (param.shape, loaded.shape, shard_id)
                param.data[start:start + length].copy_(loaded)
            return load

        def su_loader(param, loaded, shard_id=None):
            # every member of a fused module carries the same input signs (docs/FORMAT.md:31-32)
            assert loaded.shape == param.shape
            if getattr(param, "_htr_loaded", False):
                if not torch.equal(param.data.cpu(), loaded.cpu()):
                    raise ValueError("HTR: fused shards do not share the input sign vector")
                return
            param.data.copy_(loaded)
            param._htr_loaded = True

        for name, (storage, unit) in tensors.items():
            par = Parameter(storage, requires_grad=False)
            layer.register_parameter(name, par)
            set_weight_attrs(par, {"weight_loader": row_loader(unit)})
        su = Parameter(torch.empty(n // 8, dtype=torch.uint8), requires_grad=False)
        layer.register_parameter("htr_su", su)
        set_weight_attrs(su, {"weight_loader": su_loader})
        layer.htr_K = K

    def process_weights_after_loading(self, layer):
        pass

    def apply(self, layer, x, bias=None):
        from . import ops

        if _COUNT_FILE is not None:
            _census(layer, x)
        return ops.linear(x, layer.htr_qweight, layer.htr_scales, layer.htr_su, layer.htr_sv, bias)


class HTRHCLinearMethod(HTRLinearMethod):
    """Packed linear for projections whose dimensions are not multiples of 128 (htr/vllm_plugin.py:279-326 of the reference).

    spec = {"K", "m", "n", "m_pad", "n_pad"}: the stored tensors cover the zero-padded [m_pad, n_pad] matrix; the module's own
    input width is n and its output width m_out lies in [m, m_pad].  `apply` hands the unpadded activations to
    `ops.linear_padded`, which pads and slices inside the kernel.  A zero-storage uint8 `weight` buffer of the logical shape
    keeps call sites that read `.weight` for its shape working, as in the reference."""

    def __init__(self, spec):
        super().__init__(int(spec["K"]))
        self.spec = spec

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size, params_dtype,
                       **extra_weight_attrs):
        sp, K = self.spec, self.K
        n, m_out = input_size_per_partition, sum(output_partition_sizes)
        assert input_size_per_partition == input_size, "HTR: tensor parallelism is not supported"
        m_pad, n_pad = int(sp["m_pad"]), int(sp["n_pad"])
        assert n == sp["n"] and sp["m"] <= m_out <= m_pad and n <= n_pad and m_pad % 128 == 0 and n_pad % 128 == 0, (sp, n, m_out)
        assert n % 8 == 0 and m_out % 8 == 0, "HTR: padded linears need input and output widths that are multiples of 8"
        shapes = {"htr_qweight": ((m_pad // 16, n_pad // 16, 8 * K), torch.int32), "htr_scales": ((m_pad,), torch.float16),
                  "htr_su": ((n_pad // 8,), torch.uint8), "htr_sv": ((m_pad // 8,), torch.uint8)}

        def whole_loader(name):
            def load(param, loaded, shard_id=None):
                assert shard_id is None and getattr(loaded, "shard_id", None) is None, (name, shard_id)
                assert tuple(loaded.shape) == tuple(param.shape) and loaded.dtype == param.dtype, (name, param.shape, loaded.shape)
                param.data.copy_(loaded)
            return load

        for name, (shape, dt) in shapes.items():
            par = Parameter(torch.empty(shape, dtype=dt), requires_grad=False)
            layer.register_parameter(name, par)
            set_weight_attrs(par, {"weight_loader": whole_loader(name)})
        layer.htr_K = K
        layer._htr_n, layer._htr_n_pad, layer._htr_m_out, layer._htr_m_pad = n, n_pad, m_out, m_pad
        layer.register_buffer("weight", torch.zeros(1, dtype=torch.uint8).expand(m_out, n), persistent=False)
        layer._htr_weight_carrier = True

    def apply(self, layer, x, bias=None):
        from . import ops

        if _COUNT_FILE is not None:
            _census(layer, x)
            _COUNTS["hc"] += 1
        return ops.linear_padded(x, layer.htr_qweight, layer.htr_scales, layer.htr_su, layer.htr_sv, bias, m_out=layer._htr_m_out)


# optional dispatch census (htr/vllm_plugin.py:132-150): HTR_COUNT_FILE=<path> counts calls per batch bucket and width
_COUNT_FILE = os.environ.get("HTR_COUNT_FILE") or None
_COUNTS = collections.Counter()


def _census(layer, x):
    M = x.numel() // x.shape[-1]
    _COUNTS["M1" if M == 1 else ("M2-8" if M <= 8 else "M>8")] += 1
    _COUNTS[f"K{layer.htr_K}"] += 1
    if (_COUNTS["M1"] + _COUNTS["M2-8"] + _COUNTS["M>8"]) % 512 == 0:
        tmp = f"{_COUNT_FILE}.{os.getpid()}.tmp"
        with open(tmp, "w") as f:
            json.dump({"pid": os.getpid(), "t": time.time(), "counts": dict(_COUNTS)}, f)
        os.replace(tmp, f"{_COUNT_FILE}.{os.getpid()}.json")


def register():
    """vllm.general_plugins entry point.  Importing this module has already registered quant_method "htr"."""
    return None
