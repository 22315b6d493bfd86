from .dataset import OaByteDataset, OaDataLoader, OaDataLoaderConfig, OaDataset, OaDataTransform, OaOadTokenDataset  # noqa: F401
