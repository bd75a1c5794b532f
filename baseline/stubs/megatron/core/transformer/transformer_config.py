class TransformerConfig:  # annotation target only
    pass
