"""Timers, clock sampling and roofline arithmetic."""
