"""Small shared utilities (padding rules, flat parameter arenas, seeding, criteria)."""
