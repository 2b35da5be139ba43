"""Framework-wide helpers: constants, collectives wrappers, losses, metrics, profiling spans."""
