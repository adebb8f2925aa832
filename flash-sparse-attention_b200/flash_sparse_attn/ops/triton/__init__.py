"""Operator layer. The sub-package keeps the reference's name (``ops.triton``) so that callers that
import ``flash_sparse_attn.ops.triton.interface`` keep working; nothing in here uses Triton."""
