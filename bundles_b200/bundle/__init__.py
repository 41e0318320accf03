"""The bundle as the serving engine loads it: `manifest.toml` plus the two op packages."""
