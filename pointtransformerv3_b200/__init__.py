"""B200-native inference path of Point Transformer V3 behind the reference's API."""
