"""Architectures: each module registers one name of config.json `architectures` (or `architecture`)."""
from . import llama, selinex, sogutar, vapelix, zulopel  # noqa: F401
