"""Everything that spans GPUs: domains and their collectives, the box and hosts steps, the gradient reducer, the rail."""
