"""Topology, window ownership, layout routes and communication backends."""
