"""`genesis.backends.cuda_error` of the reference: turn a CUDA status code into an exception."""


def check_cuda_error(result):
    """Raises RuntimeError unless `result` (an int, a cuda-python status or a (status, value...) tuple) is success;
    returns the value(s) of a tuple."""
    status, rest = (result[0], result[1:]) if isinstance(result, tuple) else (result, ())
    code = int(getattr(status, "value", status))
    if code != 0:
        name = getattr(status, "name", None)
        raise RuntimeError(f"CUDA error {code}" + (f" ({name})" if name else ""))
    if not rest:
        return None
    return rest[0] if len(rest) == 1 else rest
