"""Helpers shared by the tests: reading a model folder into numpy for the plain implementation."""
import json
import os

import numpy as np
import torch

from pulse_infer_b200.weights import SafetensorsFile


def load_plain(folder: str):
    """(config dict, {name: float64 array}) of a model folder."""
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    weights = {n: f.tensor(n).to(torch.float64).numpy().copy() for n in f.names()}
    return cfg, weights


def random_tokens(seed: int, n: int, vocab: int) -> list:
    return [int(t) for t in np.random.RandomState(seed).randint(0, vocab, size=n)]
