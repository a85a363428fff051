"""Drop-in modules for the reference's ffa-nf4fp8 directory."""
