"""Model registry: `config.json`'s "architecture" picks the class that serves a checkpoint folder.

    model = load_model("path/to/folder", dtype="bfloat16", max_seq_len=4096)

Every class offers `forward(ids, start_pos)` (`__call__`) and the greedy `generate`.  A Llama folder holds
`config.json` with the `ModelArgs` fields (config.py) under "args" and the weights as `model.npz` in the
reference's key layout (llama3.py:219-235); the other families read `model.safetensors`.
"""
from __future__ import annotations

import json
import os


def _llama(model_dir, config, *, dtype, max_seq_len, max_batch_size, device):
    from .config import ModelArgs
    from .llama3 import Llama
    fields = dict(config.get("args", {}))
    fields.update(dtype=dtype, max_batch_size=max_batch_size)
    if max_seq_len:
        fields["max_seq_len"] = max_seq_len
    return Llama(os.path.join(model_dir, "model.npz"), ModelArgs(**fields), device=device)


def _risalix(model_dir, config, *, dtype, max_seq_len, max_batch_size, device):
    from .risalix import Risalix
    from .utils import read_safetensors
    return Risalix(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype=dtype,
                   max_seq_len=max_seq_len or 256, max_batch_size=max_batch_size, device=device)


def _rakelorn(model_dir, config, *, dtype, max_seq_len, max_batch_size, device):
    from .rakelorn import Rakelorn
    from .utils import read_safetensors
    return Rakelorn(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype=dtype,
                    max_seq_len=max_seq_len or 256, max_batch_size=max_batch_size, device=device)


def _mabedra(model_dir, config, *, dtype, max_seq_len, max_batch_size, device):
    from .mabedra import Mabedra
    from .utils import read_safetensors
    return Mabedra(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype=dtype,
                   max_seq_len=max_seq_len or 256, max_batch_size=max_batch_size, device=device)


def _debuzen(model_dir, config, *, dtype, max_seq_len, max_batch_size, device):
    from .debuzen import Debuzen
    from .utils import read_safetensors
    return Debuzen(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype=dtype,
                   max_seq_len=max_seq_len or 256, max_batch_size=max_batch_size, device=device)


ARCHITECTURES = {"Llama": _llama, "Risalix": _risalix, "Rakelorn": _rakelorn, "Mabedra": _mabedra, "Debuzen": _debuzen}


def load_model(model_dir, *, dtype: str = "float32", max_seq_len: int = 0, max_batch_size: int = 1, device: int = 0):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    arch = config.get("architecture")
    if arch not in ARCHITECTURES:
        raise ValueError(f"{model_dir}: unknown architecture {arch!r} (known: {sorted(ARCHITECTURES)})")
    return ARCHITECTURES[arch](model_dir, config, dtype=dtype, max_seq_len=max_seq_len, max_batch_size=max_batch_size,
                               device=device)
