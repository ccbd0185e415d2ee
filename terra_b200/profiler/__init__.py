"""Memory timeline, FLOP / kernel-time profilers and exposed-communication accounting."""
