"""Empty stand-in for mlx.nn (only imported for type names)."""


class Module:
    pass
