from .skills import install_skill, list_skills, uninstall_skill
