"""The identity of a loaded model: one hash over its resolved configuration and over every tensor's
name, shape and stored element type.

celeg guards session files and packed batches with ``CanonicalModelFacts::fingerprint``
(src/model/inference.cpp:74-96): the graph, the layer count, the vocabulary, the numerical policy
and every bound tensor with its shape. Here the same facts are hashed with SHA-256, so that a
logits file, a benchmark line or a bug report can be tied to the model that made it. Weights'
VALUES are not part of it (two checkpoints of one architecture and size share a fingerprint, as in
celeg); the random-weights seed is therefore named beside it where it matters.
"""
from __future__ import annotations

import hashlib
import json
from typing import Any, Mapping, Tuple


def model_fingerprint(config: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]],
                      dtypes: Mapping[str, str]) -> str:
    """``config``: the resolved configuration as config.json content; ``shapes`` / ``dtypes``: every tensor
    of the checkpoint by name. Returns 64 hexadecimal digits."""
    body = {
        "config": {key: config[key] for key in sorted(config)},
        "tensors": [[name, [int(n) for n in shapes[name]], str(dtypes.get(name, ""))] for name in sorted(shapes)],
    }
    text = json.dumps(body, sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(text.encode("utf-8")).hexdigest()
