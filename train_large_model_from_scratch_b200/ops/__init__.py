from . import oracle, native, functional, moe_ops
