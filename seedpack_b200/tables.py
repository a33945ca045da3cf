"""IQ grid tables: host construction and per-device installation (placeholder until the IQ kernels land)."""


def install(device):
    return None
