"""Import-compatible alias: `import bob; bob.sdpa_bob(...)` as with the reference package."""

from flashbob_b200.interface import sdpa_bob

__all__ = ["sdpa_bob"]
