from .base import Template, template_mapping
