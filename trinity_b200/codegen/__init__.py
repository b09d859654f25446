from .convert_module import convert_ir_to_triton  # noqa: F401
