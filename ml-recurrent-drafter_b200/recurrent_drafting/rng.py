"""Seeding of the random streams used by sampling.  Mirrors recurrent_drafting/rng.py:9-16."""
import numpy
import torch


def seed_pytorch(random_seed: int) -> None:
    torch.manual_seed(random_seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(random_seed)
    numpy.random.seed(random_seed)
