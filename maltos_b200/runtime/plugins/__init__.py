"""Runtime plugins: one module per parallel strategy or auxiliary concern."""
