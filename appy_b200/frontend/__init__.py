"""Front end: comment-preserving parse, decoration-time rewrite, loop normalisation."""
