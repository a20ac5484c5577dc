"""From a model folder to a model with its weights on the device.

Tensors are read by name.  The names and shapes a model wants come from its
parts (`Model.param_infos`); a checkpoint that lacks one, holds one nobody
wants, or holds one of another shape or of a type that cannot be used fails
with a single WeightsError that lists all of them.  The reference checks the
same things tensor by tensor while parsing GGUF (src/model.rs:562-585,
:2013-2038) and stops at the first.
"""

from __future__ import annotations

import fnmatch
import sys
from typing import Dict, Mapping, Optional, Sequence, Tuple

import torch

from ..config.llama import read_config_json
from ..errors import WeightsError
from ..models.model import Model
from ..parts.base import ParamInfo, Runtime, runtime_dtype
from ..registry import describe_model
from .safetensors_io import Checkpoint

_FLOAT_STORED = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
_INT_STORED = {"I32": torch.int32, "I64": torch.int64}


def compare_with_checkpoint(
    wanted: Mapping[str, ParamInfo], found: Mapping[str, Tuple[str, Tuple[int, ...]]], redundant: Sequence[str] = ()
) -> Optional[WeightsError]:
    """found: name -> (stored dtype name, shape).  None when everything matches.
    redundant: patterns of names that may be present without being wanted (`ModelSpec.redundant_tensors`)."""
    missing = sorted(n for n in wanted if n not in found)
    unexpected = sorted(n for n in found if n not in wanted and not any(fnmatch.fnmatchcase(n, p) for p in redundant))
    wrong_shape, wrong_dtype = [], []
    for name, info in wanted.items():
        if name not in found:
            continue
        dtype, shape = found[name]
        if tuple(shape) != tuple(info.shape):
            wrong_shape.append((name, tuple(shape), tuple(info.shape)))
        ok = dtype in (_INT_STORED if info.kind == "table" else _FLOAT_STORED)
        if not ok:
            wrong_dtype.append((name, dtype))
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return None
    lines = ["the checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong_shape:
        lines.append(
            f"  wrong shape ({len(wrong_shape)}): "
            + ", ".join(f"{n} is {list(s)}, expected {list(e)}" for n, s, e in wrong_shape)
        )
    if wrong_dtype:
        lines.append(f"  unusable type ({len(wrong_dtype)}): " + ", ".join(f"{n} is {d}" for n, d in wrong_dtype))
    return WeightsError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)


def place(tensor: torch.Tensor, info: ParamInfo, runtime: Runtime) -> torch.Tensor:
    """A stored tensor in its run type on the run's device."""
    target = runtime_dtype(info, tensor.dtype, runtime.dtype)
    return tensor.to(device=runtime.device, dtype=target).contiguous()


def load_tensors(model: Model, source: Mapping[str, torch.Tensor] | Checkpoint) -> None:
    """Check `source` against the model, move the tensors and hand them to the parts."""
    wanted = model.param_infos()
    if isinstance(source, Checkpoint):
        found = {n: (source.info(n).dtype, source.info(n).shape) for n in source.names()}
        read = source.read
    else:
        rev = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64"}
        found = {n: (rev.get(t.dtype, str(t.dtype)), tuple(t.shape)) for n, t in source.items()}
        read = source.__getitem__
    redundant = tuple(model.spec.redundant_tensors)
    err = compare_with_checkpoint(wanted, found, redundant)
    if err is not None:
        raise err
    passed_over = sorted(n for n in found if n not in wanted)
    if passed_over:
        print(f"[rusty_llama_b200] passing over {len(passed_over)} tensors the model recomputes or shares: "
              + ", ".join(passed_over[:4]) + (" ..." if len(passed_over) > 4 else ""), file=sys.stderr)
    placed: Dict[str, torch.Tensor] = {}
    for name, info in wanted.items():
        placed[name] = place(read(name), info, model.rt)
    model.load(placed)


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Model:
    """config.json picks the architecture and the sizes, model.safetensors gives the weights."""
    spec = describe_model(read_config_json(model_dir))
    runtime = Runtime.create(device, dtype)
    model = Model(spec, runtime)
    with Checkpoint(model_dir) as ckpt:
        load_tensors(model, ckpt)
    return model
