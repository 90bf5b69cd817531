"""Python surface mirroring aqt.jax.v2 (config, aqt_dot_general, aqt_quantizer, ...)."""
