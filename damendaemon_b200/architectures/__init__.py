"""One module per architecture: config -> ModelSpec, checkpoint names, random init."""
