"""Per-layer digests of a model's residual stream, for finding the layer where two runs part ways.

    from r4dx_b200.utils.probe import LayerDigests
    d = LayerDigests.attach(model)          # eager calls only (graph replays do not call the probe)
    model.feed(ids); rows = d.rows          # [{"call": 0, "layer": 3, "rows": 4, "mean": .., "absmax": .., "l2": ..}, ...]
    LayerDigests.first_difference(a.rows, b.rows, rel=1e-3)

(reference: src/model/debug_probe.h keeps per-layer probes and state digests for the same purpose.)
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import torch


class LayerDigests:
    def __init__(self):
        self.rows: List[Dict[str, float]] = []
        self.call = -1
        self._last_layer = 1 << 30

    @staticmethod
    def attach(model) -> "LayerDigests":
        d = LayerDigests()
        model.probe = d
        return d

    def __call__(self, layer: int, x: torch.Tensor) -> None:
        if layer <= self._last_layer:
            self.call += 1
        self._last_layer = layer
        f = x.float()
        self.rows.append({"call": self.call, "layer": int(layer), "rows": int(x.shape[0]), "mean": float(f.mean()),
                          "absmax": float(f.abs().max()), "l2": float(f.pow(2).sum().sqrt())})

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            for r in self.rows:
                f.write(json.dumps(r) + "\n")

    @staticmethod
    def first_difference(a: List[Dict[str, float]], b: List[Dict[str, float]], rel: float = 1e-3) -> Optional[Dict[str, float]]:
        """The first (call, layer) at which the two digest lists differ by more than ``rel`` of the larger l2 norm."""
        for ra, rb in zip(a, b):
            if (ra["call"], ra["layer"], ra["rows"]) != (rb["call"], rb["layer"], rb["rows"]):
                return {"call": ra["call"], "layer": ra["layer"], "reason": "different call sequence"}
            ref = max(abs(ra["l2"]), abs(rb["l2"]), 1e-30)
            if abs(ra["l2"] - rb["l2"]) > rel * ref or abs(ra["absmax"] - rb["absmax"]) > rel * max(ra["absmax"], rb["absmax"], 1e-30):
                return {"call": ra["call"], "layer": ra["layer"], "l2_a": ra["l2"], "l2_b": rb["l2"]}
        return None
