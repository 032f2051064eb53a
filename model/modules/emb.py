from train_large_model_from_scratch_b200.models.modules.emb import TextEmbedding, ImgEmbedding  # noqa: F401
