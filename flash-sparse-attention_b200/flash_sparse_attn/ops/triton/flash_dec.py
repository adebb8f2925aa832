"""Host launcher of the decode pass (filled in by the decode kernels)."""


def attn_decode(kind, *args, **kwargs):
    raise NotImplementedError("decode kernels are not built yet")
