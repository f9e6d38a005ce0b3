"""B200-native OAL causal grouped-quadratic attention."""
