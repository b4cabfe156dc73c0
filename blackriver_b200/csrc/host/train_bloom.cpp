// placeholder main until the driver is written
int main() { return 0; }
