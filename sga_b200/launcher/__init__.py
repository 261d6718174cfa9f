"""Job launcher: yaml -> flags -> per-host torchrun scripts over ssh."""
