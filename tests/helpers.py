"""Shared small configurations for CPU tests."""

from dataclasses import replace

import numpy as np

from lyra_b200.variants import model_variant


def small_config(**kw):
    """The ``dev`` variant with a small vocabulary so CPU steps take milliseconds."""
    base = replace(model_variant("dev"), seq_len=32, vocab_size=500, padded_vocab_size=512, n_layers=4,
                   mlp_map=("dense", "moe", "dense", "moe"), implementation="torch")
    return replace(base, **kw)


def token_file(path, n=6000, vocab=500, seed=0):
    np.save(path, np.random.default_rng(seed).integers(0, vocab, size=n).astype("<i4"))
    return path


def free_port() -> int:
    """A port that is free right now, drawn from below the kernel's ephemeral range: ports the OS hands out itself (bind to 0)
    come from the range that the collectives library's own sockets use, and a spawned rank has then found its rendezvous port
    taken."""
    import random
    import socket

    for _ in range(200):
        port = random.randint(12000, 29999)
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
            try:
                sock.bind(("127.0.0.1", port))
            except OSError:
                continue
            return port
    raise RuntimeError("no free port found")
