"""Roll-out worker helpers (prompt store + vLLM server launcher).  Not connected to
the trainer, as in the reference (rl/worker_node)."""
