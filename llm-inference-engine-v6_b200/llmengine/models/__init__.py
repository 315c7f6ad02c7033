"""Architectures: each module registers one name of config.json `architectures` (or `architecture`)."""
from . import llama, selinex, vapelix, zulopel  # noqa: F401
