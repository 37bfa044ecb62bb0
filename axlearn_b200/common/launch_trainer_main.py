"""``python -m axlearn_b200.common.launch_trainer_main --module=text.gpt.c4_trainer --config=fuji-test-v1
--trainer_dir=/tmp/run`` (reference: axlearn/common/launch_trainer_main.py)."""

from axlearn_b200.common.launch_trainer import main

if __name__ == "__main__":
    main()
