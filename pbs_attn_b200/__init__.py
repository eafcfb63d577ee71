"""B200-native (sm_100a) implementation of the PBS-Attn prefill hot path."""
