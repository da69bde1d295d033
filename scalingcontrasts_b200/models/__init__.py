"""torch modules: the loss module with its learnable temperature and bias, and the projector tower."""
