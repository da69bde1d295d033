"""Host-side utilities: keyed inputs, timing, clocks sampling, status decoding, checkpoints."""
