"""Python front end of the tcgen05 GEMM (filled in with the kernel)."""


def supported(x, w) -> bool:
    return False


def gemm_nt(x, w, bias=None, out=None):
    raise NotImplementedError
