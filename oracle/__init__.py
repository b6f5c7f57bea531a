"""CPU oracle: test infrastructure only (see cpu_ref.c)."""
