"""Checkpoint directories in the Hugging Face layout (config.json + *.safetensors or *.bin shards),
as the reference's command line loads them (recurrent_drafting/cmd/generate.py:55-72,
modeling_drafter.py:23-30).  Tensors are read one at a time, so a 7B or 13B checkpoint is packed into
the kernels' weight layouts without a second full copy in host memory."""
import json
import os
from typing import Dict, Iterator, List

import torch


class LazyCheckpoint:
    """Name -> tensor view of a checkpoint directory.  `pop(name)` loads that tensor from its shard;
    iterating yields the names not taken yet."""

    def __init__(self, path: str):
        self.path = path
        self._where: Dict[str, str] = {}
        index = [f for f in ("model.safetensors.index.json", "pytorch_model.bin.index.json") if os.path.exists(os.path.join(path, f))]
        if index:
            with open(os.path.join(path, index[0])) as f:
                self._where = dict(json.load(f)["weight_map"])
        else:
            files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors")) or sorted(
                f for f in os.listdir(path) if f.endswith(".bin"))
            if not files:
                raise FileNotFoundError(f"no *.safetensors or *.bin weights under {path}")
            for fn in files:
                for name in self._names_of(fn):
                    self._where[name] = fn
        self._bin_cache: Dict[str, Dict[str, torch.Tensor]] = {}

    def _names_of(self, fn: str) -> List[str]:
        full = os.path.join(self.path, fn)
        if fn.endswith(".safetensors"):
            from safetensors import safe_open

            with safe_open(full, framework="pt", device="cpu") as f:
                return list(f.keys())
        self._bin_cache[fn] = torch.load(full, map_location="cpu", weights_only=True)
        return list(self._bin_cache[fn].keys())

    def __iter__(self) -> Iterator[str]:
        return iter(list(self._where))

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def __len__(self) -> int:
        return len(self._where)

    def keys(self):
        return list(self._where)

    def pop(self, name: str) -> torch.Tensor:
        fn = self._where.pop(name)
        full = os.path.join(self.path, fn)
        if fn.endswith(".safetensors"):
            from safetensors import safe_open

            with safe_open(full, framework="pt", device="cpu") as f:
                return f.get_tensor(name)
        if fn not in self._bin_cache:
            self._bin_cache[fn] = torch.load(full, map_location="cpu", weights_only=True)
        return self._bin_cache[fn].pop(name)


def save_directory(path: str, config, state_dict: Dict[str, torch.Tensor]) -> None:
    """config.json + model.safetensors under `path`."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    config.save_pretrained(path)
    save_file({k: v.detach().cpu().contiguous() for k, v in state_dict.items()}, os.path.join(path, "model.safetensors"))
