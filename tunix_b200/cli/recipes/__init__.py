"""Dataset recipes of the CLI (tunix/cli/recipes)."""
