"""Reference module path ``ipex_llm.utils.ipex_importer`` (python/llm/src/ipex_llm/utils/ipex_importer.py:35-173):
the reference imports Intel Extension for PyTorch before anything else.  There is no such dependency here; the
importer keeps its interface and reports that nothing was imported."""


class IPEXImporter:
    def __init__(self):
        self.ipex_version = None

    @staticmethod
    def is_xpu_version_installed() -> bool:
        return False

    def import_ipex(self):
        return None

    def get_ipex_version(self):
        return None


ipex_importer = IPEXImporter()
