"""Inputs of the tests: the seeded generators of the package (the benchmark uses the same ones)
and the helper that sets the library's test hook."""
from torch_points_kernels_b200.synthetic import *  # noqa: F401,F403


def use_paths(monkeypatch, *tokens):
    """Sets TPK_B200_TEST, the one environment variable the library reads, to the given
    `name` / `name=value` tokens (None entries are dropped; no token clears it)."""
    tokens = [t for t in tokens if t]
    if tokens:
        monkeypatch.setenv("TPK_B200_TEST", ",".join(tokens))
    else:
        monkeypatch.delenv("TPK_B200_TEST", raising=False)
