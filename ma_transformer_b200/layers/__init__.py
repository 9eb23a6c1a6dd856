"""nn.Module surface, named after the reference's src/layers package."""
